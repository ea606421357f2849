// moe_align for sm_100a: warp-aggregated histogram -> scan -> stable scatter.
//
// Contract (same outputs as pi::moe_align, prime_moe/csrc/kernels/fused_moe_bf16_kernel.cu:853-928):
//   sorted_token_ids[max_padded]: for every expert its pair ids followed by -1 up to a multiple of
//   pad_to, experts in ascending order, -1 after num_tokens_post_padded;
//   expert_ids[max_blocks]: expert owning each block_m-row block (largest e with offs[e] <= row),
//   num_experts-1 for blocks past the end; num_tokens_post_padded[0] = sum of padded counts.
// The reference runs ONE CTA with shared-memory atomics and a serial scan, and leaves the order
// inside an expert to the atomics. Here the ids are cut into contiguous per-warp segments; a warp
// counts its segment with __match_any_sync groups (counters private to the warp, in shared memory),
// the per-CTA sums go to a small counts[cta][expert] matrix, and the scatter pass - which scans that
// matrix itself - replays the segments in order, so the result is deterministic and ascending inside
// each expert.
//
// HBM traffic: 4n bytes of ids read (a second time from L2), 4*max_padded written twice at most
// (-1 fill + scatter), plus the (#CTAs <= #SMs) x E counter matrix (scratch).
#include <stdio.h>

#include <algorithm>

#include "host_common.h"
#include "route_warp.cuh"

namespace pmoe {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;
constexpr int kSmallN = 4096;      // up to here a single CTA of 8 warps does everything, no scratch
constexpr int kSmallN32 = 16384;   // ... and up to here a single CTA of 32 warps, when its counters fit (E <= 256)
constexpr int kMaxExperts = 1024;

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// Count the ids of [begin, end) into cnt[0..E) (private to the calling warp, already zeroed).
// Four 32-id groups are loaded ahead of their match rounds so that the loads overlap.
__device__ __forceinline__ void warp_histogram(const int32_t *__restrict__ ids, int begin, int end, int E,
                                               int *cnt) {
    const int lane = threadIdx.x & 31;
    for (int base = begin; base < end; base += 128) {
        int v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = base + 32 * u + lane;
            v[u] = (i < end) ? __ldg(ids + i) : -1;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (base + 32 * u >= end) break;     // uniform per warp
            int id = v[u];
            const bool valid = id >= 0 && id < E;
            if (!valid) id = -1;
            const unsigned peers = __match_any_sync(0xffffffffu, id);
            if (valid && (peers & lanemask_lt()) == 0) cnt[id] += __popc(peers);
            __syncwarp();
        }
    }
}

// Replay [begin, end): cur[e] is this warp's next write position for expert e.
__device__ __forceinline__ void warp_scatter(const int32_t *__restrict__ ids, int begin, int end, int E,
                                             int *cur, int32_t *__restrict__ sorted, int max_padded) {
    const int lane = threadIdx.x & 31;
    for (int base = begin; base < end; base += 128) {
        int v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = base + 32 * u + lane;
            v[u] = (i < end) ? __ldg(ids + i) : -1;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (base + 32 * u >= end) break;     // uniform per warp
            const int i = base + 32 * u + lane;
            int id = v[u];
            const bool valid = id >= 0 && id < E;
            if (!valid) id = -1;
            const unsigned peers = __match_any_sync(0xffffffffu, id);
            const int rank = __popc(peers & lanemask_lt());
            int pos = 0;
            if (valid) pos = cur[id] + rank;
            __syncwarp();
            if (valid) {
                if (pos < max_padded) sorted[pos] = i;
                if (rank == 0) cur[id] += __popc(peers);
            }
            __syncwarp();
        }
    }
}

__device__ __forceinline__ int find_expert(const int *offs, int E, int row) {
    int lo = 0, hi = E - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (offs[mid] <= row) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

// Exclusive scan of padded totals over E experts by one CTA: tot[e] (shared) -> offs[e], offs[E].
// `wsum` holds blockDim/32 ints. All threads of the CTA call this.
__device__ void block_offsets(const int *tot, int *offs, int *wsum, int E, int pad_to) {
    const int nthr = blockDim.x;
    const int per = (E + nthr - 1) / nthr;  // consecutive experts per thread
    const int e0 = threadIdx.x * per;
    int local = 0;
    for (int k = 0; k < per; ++k) {
        const int e = e0 + k;
        if (e < E) local += (tot[e] + pad_to - 1) / pad_to * pad_to;
    }
    int incl = local;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int nw = nthr >> 5;
        int v = lane < nw ? wsum[lane] : 0;
        int s = v;
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, s, d);
            if (lane >= d) s += u;
        }
        if (lane < nw) wsum[lane] = s - v;  // exclusive over warps
        if (lane == 31) offs[E] = s;        // grand total
    }
    __syncthreads();
    int run = wsum[warp] + incl - local;
    for (int k = 0; k < per; ++k) {
        const int e = e0 + k;
        if (e < E) {
            offs[e] = run;
            run += (tot[e] + pad_to - 1) / pad_to * pad_to;
        }
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------
// small n: one CTA, no scratch
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) moe_align_small_kernel(
    const int32_t *__restrict__ ids, int32_t *__restrict__ sorted, int32_t *__restrict__ expert_ids,
    int32_t *__restrict__ npp, int n, int E, int block_m, int pad_to, int max_padded, int max_blocks) {
    extern __shared__ int sm[];
    const int nthr = blockDim.x, nwarps = nthr >> 5;   // 8 warps, or 32 for the larger single-CTA problems
    int *cnt = sm;                 // [nwarps][E]
    int *tot = cnt + nwarps * E;   // [E]
    int *offs = tot + E;           // [E + 1]
    int *wsum = offs + E + 1;      // [nwarps]
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < nwarps * E; i += nthr) cnt[i] = 0;
    __syncthreads();
    const int seg = ((n + nwarps - 1) / nwarps + 31) & ~31;
    const int begin = min(warp * seg, n), end = min(begin + seg, n);
    warp_histogram(ids, begin, end, E, cnt + warp * E);
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += nthr) {
        int run = 0;
        for (int w = 0; w < nwarps; ++w) {
            const int c = cnt[w * E + e];
            cnt[w * E + e] = run;
            run += c;
        }
        tot[e] = run;
    }
    __syncthreads();
    block_offsets(tot, offs, wsum, E, pad_to);
    const int total = offs[E];
    if (threadIdx.x == 0) npp[0] = total;
    {   // -1 fill, 16 bytes per store (sorted_token_ids is 16-byte aligned)
        int4 *s4 = reinterpret_cast<int4 *>(sorted);
        const int n4 = max_padded >> 2;
        const int4 m1 = make_int4(-1, -1, -1, -1);
        for (int i = threadIdx.x; i < n4; i += nthr) s4[i] = m1;
        if (threadIdx.x < (max_padded & 3)) sorted[(n4 << 2) + threadIdx.x] = -1;
    }
    for (int j = threadIdx.x; j < max_blocks; j += nthr) {
        const int row = j * block_m;
        expert_ids[j] = row >= total ? E - 1 : find_expert(offs, E, row);
    }
    for (int e = threadIdx.x; e < E; e += nthr) {
        const int o = offs[e];
        for (int w = 0; w < nwarps; ++w) cnt[w * E + e] += o;
    }
    __syncthreads();  // orders the -1 fill before the scatter stores of this CTA
    warp_scatter(ids, begin, end, E, cnt + warp * E, sorted, max_padded);
}

// ---------------------------------------------------------------------------------------------
// general n: two launches. The ids are cut into one contiguous segment per CTA (and per warp inside it).
//   histogram kernel   per-warp private counters in shared memory -> counts[cta][e] (coalesced), and the
//                      -1 fill of sorted_token_ids
//   scatter kernel     every CTA rebuilds its per-warp counters (its ids come back from L2), reads the
//                      counts of ALL CTAs - at most #SM x E integers, L2-resident - to get each expert's
//                      total and the number of its ids in lower CTAs, scans the padded totals itself and
//                      replays its segment. The scan is thus done redundantly by every CTA instead of by a
//                      one-CTA kernel in between; expert_ids is written by all CTAs in turns, npp by CTA 0.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) moe_align_hist_kernel(
    const int32_t *__restrict__ ids, int n, int E, int seg, int *__restrict__ counts,
    int32_t *__restrict__ sorted, int max_padded) {
    extern __shared__ int sm[];
    // the scatter kernel may start its own counting pass now; it waits for this whole grid before it reads the
    // counts or writes sorted_token_ids
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < kWarpsPerCta * E; i += kThreads) sm[i] = 0;
    __syncthreads();
    const int gw = blockIdx.x * kWarpsPerCta + warp;
    const int begin = min(gw * seg, n), end = min(begin + seg, n);
    warp_histogram(ids, begin, end, E, sm + warp * E);
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += kThreads) {
        int t = 0;
#pragma unroll
        for (int w = 0; w < kWarpsPerCta; ++w) t += sm[w * E + e];
        counts[static_cast<size_t>(blockIdx.x) * E + e] = t;
    }
    // -1 everywhere; the scatter kernel (later in stream order) overwrites the valid slots
    int4 *s4 = reinterpret_cast<int4 *>(sorted);
    const int n4 = max_padded >> 2;
    const int4 m1 = make_int4(-1, -1, -1, -1);
    for (int i = blockIdx.x * kThreads + threadIdx.x; i < n4; i += gridDim.x * kThreads) s4[i] = m1;
    if (blockIdx.x == 0 && threadIdx.x < (max_padded & 3)) sorted[(n4 << 2) + threadIdx.x] = -1;
}

__global__ void __launch_bounds__(kThreads) moe_align_scatter_kernel(
    const int32_t *__restrict__ ids, int n, int E, int seg, const int *__restrict__ counts, int block_m,
    int pad_to, int32_t *__restrict__ sorted, int32_t *__restrict__ expert_ids, int32_t *__restrict__ npp,
    int max_padded, int max_blocks, int ids_from_primary) {
    extern __shared__ int sm[];
    int *cnt = sm;                       // [kWarpsPerCta][E] per-warp counts, later per-warp write cursors
    int *tot = cnt + kWarpsPerCta * E;   // [E] ids of expert e in all CTAs
    int *pre = tot + E;                  // [E] ids of expert e in lower CTAs
    int *offs = pre + E;                 // [E + 1]
    int *wsum = offs + E + 1;            // [kWarpsPerCta]
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < kWarpsPerCta * E + 2 * E; i += kThreads) sm[i] = 0;
    __syncthreads();
    const int gw = blockIdx.x * kWarpsPerCta + warp;
    const int begin = min(gw * seg, n), end = min(begin + seg, n);
    // after the fused router the ids themselves come from the preceding kernel: wait before reading them
    if (ids_from_primary) asm volatile("griddepcontrol.wait;" ::: "memory");
    warp_histogram(ids, begin, end, E, cnt + warp * E);
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the histogram kernel's counts and -1 fill are complete
    // column sums of counts[cta][e]: `parts` threads share one expert when there are fewer experts than threads
    const int ctas = gridDim.x, me = blockIdx.x;
    const int parts = max(1, kThreads / E);
    for (int idx = threadIdx.x; idx < E * parts; idx += kThreads) {   // consecutive threads, consecutive experts
        const int e = idx % E, part = idx / E;
        int t = 0, p = 0;
#pragma unroll 8
        for (int c = part; c < ctas; c += parts) {
            const int v = __ldg(counts + static_cast<size_t>(c) * E + e);
            t += v;
            p += c < me ? v : 0;
        }
        atomicAdd(&tot[e], t);   // shared-memory integer adds: the sum does not depend on their order
        atomicAdd(&pre[e], p);
    }
    __syncthreads();
    block_offsets(tot, offs, wsum, E, pad_to);
    const int total = offs[E];
    if (me == 0 && threadIdx.x == 0) npp[0] = total;
    for (int j = me * kThreads + threadIdx.x; j < max_blocks; j += ctas * kThreads) {
        const int row = j * block_m;
        expert_ids[j] = row >= total ? E - 1 : find_expert(offs, E, row);
    }
    for (int e = threadIdx.x; e < E; e += kThreads) {
        int run = offs[e] + pre[e];
#pragma unroll
        for (int w = 0; w < kWarpsPerCta; ++w) {
            const int c = cnt[w * E + e];
            cnt[w * E + e] = run;
            run += c;
        }
    }
    __syncthreads();
    warp_scatter(ids, begin, end, E, cnt + warp * E, sorted, max_padded);
}

struct Plan {
    int ctas;       // grid of the histogram / scatter kernels (0 = single-CTA path)
    int seg;        // ids per warp (multiple of 32)
    size_t ws_ints; // scratch ints: counts[ctas][E]
};

constexpr int kIdsPerCtaMin = 2048;

Plan make_plan(int n, int E) {
    Plan p{};
    if (n <= kSmallN || (n <= kSmallN32 && E <= 256)) return p;
    int ctas = (n + kIdsPerCtaMin - 1) / kIdsPerCtaMin;
    ctas = std::max(1, std::min(ctas, sm_count()));
    p.ctas = ctas;
    const int warps = ctas * kWarpsPerCta;
    p.seg = ((n + warps - 1) / warps + 31) & ~31;
    p.ws_ints = static_cast<size_t>(E) * ctas;
    return p;
}

int check_args(const void *topk_ids, const void *sorted, const void *expert_ids, const void *npp, int n, int E,
               int block_m, int pad_to, int max_padded, int max_blocks) {
    PMOE_REQUIRE(topk_ids && sorted && expert_ids && npp, PMOE_ERR_BAD_ARG, "moe_align: null pointer");
    PMOE_REQUIRE(n >= 0 && E > 0 && block_m > 0 && pad_to > 0, PMOE_ERR_BAD_ARG,
                 "moe_align: n >= 0, num_experts > 0, block_m > 0 and pad_to > 0 required");
    PMOE_REQUIRE(E <= kMaxExperts, PMOE_ERR_UNSUPPORTED, "moe_align supports at most 1024 experts, got %d", E);
    PMOE_REQUIRE(pad_to % block_m == 0, PMOE_ERR_BAD_ARG, "moe_align: pad_to must be a multiple of block_m");
    const long long need = (static_cast<long long>(n) + static_cast<long long>(E) * (pad_to - 1) + pad_to - 1) /
                           pad_to * pad_to;
    PMOE_REQUIRE(max_padded >= need, PMOE_ERR_BAD_ARG, "moe_align: max_padded %d < required %lld", max_padded,
                 need);
    PMOE_REQUIRE(static_cast<long long>(max_blocks) * block_m >= max_padded, PMOE_ERR_BAD_ARG,
                 "moe_align: max_blocks %d does not cover max_padded %d", max_blocks, max_padded);
    PMOE_REQUIRE((reinterpret_cast<uintptr_t>(sorted) & 15) == 0, PMOE_ERR_BAD_ARG,
                 "moe_align: sorted_token_ids must be 16-byte aligned");
    return PMOE_OK;
}

int launch(const int32_t *topk_ids, int32_t *sorted, int32_t *expert_ids, int32_t *npp, int n, int E,
           int block_m, int pad_to, int max_padded, int max_blocks, const Plan &p, int *ws,
           cudaStream_t stream) {
    if (p.ctas == 0) {
        const int warps = n > 1024 && E <= 256 ? 32 : kWarpsPerCta;
        const size_t smem = (static_cast<size_t>(warps) * E + 2 * E + 1 + warps) * sizeof(int);   // <= 35 KB
        moe_align_small_kernel<<<1, warps * 32, smem, stream>>>(topk_ids, sorted, expert_ids, npp, n, E, block_m,
                                                             pad_to, max_padded, max_blocks);
        PMOE_CUDA_OK(cudaGetLastError());
        return PMOE_OK;
    }
    int *counts = ws;
    const size_t smem_h = static_cast<size_t>(kWarpsPerCta) * E * sizeof(int);
    moe_align_hist_kernel<<<p.ctas, kThreads, smem_h, stream>>>(topk_ids, n, E, p.seg, counts, sorted, max_padded);
    PMOE_CUDA_OK(cudaGetLastError());
    const size_t smem_s = (static_cast<size_t>(kWarpsPerCta) * E + 3 * static_cast<size_t>(E) + 1 + kWarpsPerCta) *
                          sizeof(int);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_s;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, moe_align_scatter_kernel, topk_ids, n, E, p.seg, static_cast<const int *>(counts),
                                    block_m, pad_to, sorted, expert_ids, npp, max_padded, max_blocks, 0));
    return PMOE_OK;
}

}  // namespace
}  // namespace pmoe

// ---------------------------------------------------------------------------------------------
// router fused with the histogram pass: one kernel routes the tokens (softmax + top-k, one warp per token,
// route_warp.cuh), writes topk_ids / topk_weights, counts its own ids per expert and fills sorted_token_ids with
// -1 - i.e. it replaces route_topk_kernel AND moe_align_hist_kernel, and the ids are not read back for counting.
// CTA c owns the ids [c*8*seg, (c+1)*8*seg) of the align plan, i.e. 8*seg / top_k whole tokens (the entry point
// falls back to the two separate kernels when top_k does not divide 8*seg). 32 warps per CTA: the grid is the
// align plan's (<= #SMs CTAs), so the tokens of a CTA are spread over more warps than the histogram pass has.
// ---------------------------------------------------------------------------------------------
namespace pmoe {
namespace {

template <typename T, int PER>
__global__ void __launch_bounds__(1024) route_hist_kernel(
    const T *__restrict__ logits, int tokens, int E, int top_k, int renormalize, int32_t *__restrict__ topk_ids,
    float *__restrict__ topk_weights, int tokens_per_cta, int *__restrict__ counts, int32_t *__restrict__ sorted,
    int max_padded) {
    extern __shared__ int s_cnt[];   // [E]
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int e = threadIdx.x; e < E; e += blockDim.x) s_cnt[e] = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int t0 = blockIdx.x * tokens_per_cta, t1 = min(tokens, t0 + tokens_per_cta);
    for (int t = t0 + warp; t < t1; t += nwarps) {
        int idx;
        float w;
        route_token_warp<T, PER>(logits + static_cast<size_t>(t) * E, E, top_k, renormalize, lane, idx, w);
        if (lane < top_k) {
            topk_ids[static_cast<size_t>(t) * top_k + lane] = idx;
            topk_weights[static_cast<size_t>(t) * top_k + lane] = w;
            atomicAdd(&s_cnt[idx], 1);   // shared-memory integer counts: independent of the order of the adds
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[static_cast<size_t>(blockIdx.x) * E + e] = s_cnt[e];
    int4 *s4 = reinterpret_cast<int4 *>(sorted);
    const int n4 = max_padded >> 2;
    const int4 m1 = make_int4(-1, -1, -1, -1);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) s4[i] = m1;
    if (blockIdx.x == 0 && threadIdx.x < (max_padded & 3)) sorted[(n4 << 2) + threadIdx.x] = -1;
}

template <typename T>
int launch_route_hist(const T *logits, int tokens, int E, int top_k, int renormalize, int32_t *ids, float *wts,
                      const Plan &p, int *counts, int32_t *sorted, int max_padded, cudaStream_t stream) {
    const int tokens_per_cta = kWarpsPerCta * p.seg / top_k;
    const size_t smem = static_cast<size_t>(E) * sizeof(int);
    const int per = (E + 31) / 32;
#define PMOE_ROUTE_HIST_CASE(P)                                                                                      \
    if (per <= P) {                                                                                                  \
        route_hist_kernel<T, P><<<p.ctas, 1024, smem, stream>>>(logits, tokens, E, top_k, renormalize, ids, wts,     \
                                                               tokens_per_cta, counts, sorted, max_padded);         \
        PMOE_CUDA_OK(cudaGetLastError());                                                                            \
        return PMOE_OK;                                                                                              \
    }
    PMOE_ROUTE_HIST_CASE(1)
    PMOE_ROUTE_HIST_CASE(2)
    PMOE_ROUTE_HIST_CASE(4)
    PMOE_ROUTE_HIST_CASE(8)
    PMOE_ROUTE_HIST_CASE(16)
    PMOE_ROUTE_HIST_CASE(32)
#undef PMOE_ROUTE_HIST_CASE
    return set_error(PMOE_ERR_UNSUPPORTED, "route_topk_align supports at most 1024 experts, got %d", E);
}

}  // namespace
}  // namespace pmoe

extern "C" int pmoe_route_topk_align(const void *logits, int logits_dtype, int T, int num_experts, int top_k,
                                     int renormalize, int32_t *topk_ids, float *topk_weights,
                                     int32_t *sorted_token_ids, int32_t *expert_ids, int32_t *num_tokens_post_padded,
                                     int block_m, int pad_to, int max_padded, int max_blocks, void *workspace,
                                     size_t workspace_bytes, pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(T >= 0 && top_k > 0 && static_cast<long long>(T) * top_k < (1ll << 31), PMOE_ERR_BAD_ARG,
                 "route_topk_align: T >= 0, top_k > 0 and T * top_k < 2^31 required");
    const int n = T * top_k;
    if (int rc = check_args(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, n, num_experts, block_m,
                            pad_to, max_padded, max_blocks))
        return rc;
    const Plan p = make_plan(n, num_experts);
    PMOE_REQUIRE(p.ws_ints == 0 || (workspace && workspace_bytes >= p.ws_ints * sizeof(int)), PMOE_ERR_BAD_ARG,
                 "route_topk_align: workspace of %zu bytes required, got %zu", p.ws_ints * sizeof(int), workspace_bytes);
    const bool fused = p.ctas > 0 && (kWarpsPerCta * p.seg) % top_k == 0 && logits && topk_weights && top_k <= 32 &&
                       top_k <= num_experts && num_experts <= kMaxExperts &&
                       (logits_dtype == PMOE_DTYPE_F32 || logits_dtype == PMOE_DTYPE_BF16);
    if (!fused) {   // small problems (one CTA aligns them) and top_k that does not divide a CTA's id range
        if (int rc = pmoe_route_topk(logits, logits_dtype, T, num_experts, top_k, renormalize, topk_ids, topk_weights,
                                     stream))
            return rc;
        return launch(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, n, num_experts, block_m, pad_to,
                      max_padded, max_blocks, p, static_cast<int *>(workspace), stream);
    }
    int *counts = static_cast<int *>(workspace);
    int rc = logits_dtype == PMOE_DTYPE_F32
                 ? launch_route_hist(static_cast<const float *>(logits), T, num_experts, top_k, renormalize ? 1 : 0,
                                     topk_ids, topk_weights, p, counts, sorted_token_ids, max_padded, stream)
                 : launch_route_hist(static_cast<const __nv_bfloat16 *>(logits), T, num_experts, top_k,
                                     renormalize ? 1 : 0, topk_ids, topk_weights, p, counts, sorted_token_ids,
                                     max_padded, stream);
    if (rc) return rc;
    const size_t smem_s = (static_cast<size_t>(kWarpsPerCta) * num_experts + 3 * static_cast<size_t>(num_experts) + 1 +
                           kWarpsPerCta) * sizeof(int);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_s;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, moe_align_scatter_kernel, static_cast<const int32_t *>(topk_ids), n, num_experts,
                                    p.seg, static_cast<const int *>(counts), block_m, pad_to, sorted_token_ids, expert_ids,
                                    num_tokens_post_padded, max_padded, max_blocks, 1));
    return PMOE_OK;
}

extern "C" size_t pmoe_moe_align_workspace_bytes(int n, int num_experts) {
    if (n < 0 || num_experts <= 0) return 0;
    return pmoe::make_plan(n, num_experts).ws_ints * sizeof(int);
}

extern "C" int pmoe_moe_align_ws(const int32_t *topk_ids, int32_t *sorted_token_ids, int32_t *expert_ids,
                                 int32_t *num_tokens_post_padded, int n, int num_experts, int block_m,
                                 int pad_to, int max_padded, int max_blocks, void *workspace,
                                 size_t workspace_bytes, pmoe_stream_t stream) {
    using namespace pmoe;
    if (int rc = check_args(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, n, num_experts,
                            block_m, pad_to, max_padded, max_blocks))
        return rc;
    const Plan p = make_plan(n, num_experts);
    PMOE_REQUIRE(p.ws_ints == 0 || (workspace && workspace_bytes >= p.ws_ints * sizeof(int)), PMOE_ERR_BAD_ARG,
                 "moe_align: workspace of %zu bytes required, got %zu", p.ws_ints * sizeof(int),
                 workspace_bytes);
    return launch(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, n, num_experts, block_m,
                  pad_to, max_padded, max_blocks, p, static_cast<int *>(workspace), stream);
}

extern "C" int pmoe_moe_align(const int32_t *topk_ids, int32_t *sorted_token_ids, int32_t *expert_ids,
                              int32_t *num_tokens_post_padded, int n, int num_experts, int block_m, int pad_to,
                              int max_padded, int max_blocks, pmoe_stream_t stream) {
    using namespace pmoe;
    if (int rc = check_args(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, n, num_experts,
                            block_m, pad_to, max_padded, max_blocks))
        return rc;
    const Plan p = make_plan(n, num_experts);
    int *ws = nullptr;
    if (p.ws_ints)
        if (int rc = scratch_alloc(reinterpret_cast<void **>(&ws), p.ws_ints * sizeof(int), stream)) return rc;
    const int rc = launch(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, n, num_experts,
                          block_m, pad_to, max_padded, max_blocks, p, ws, stream);
    if (ws)
        if (int rc2 = scratch_free(ws, stream)) return rc2;
    return rc;
}

// ---------------------------------------------------------------------------------------------
// moe_align for callers that must not allocate
// ---------------------------------------------------------------------------------------------
// Some hosts of this library cannot call cudaMalloc (or any allocator) at the point where routing
// runs: an inference server whose memory budget is fixed after start-up and which forbids further
// driver allocations, a plugin running inside another framework's stream callback or allocator
// hook, a process whose whole device memory has already been handed to a pool it does not own.
// For them the per-CTA counter matrix lives in a fixed array that is part of
// the library image. Every GPU that loads the library carries these 256 KiB until the process exits.
#define PMOE_STATIC_SCRATCH_INTS (1u << 16)  /* 256 KiB: the stated maximum */
static __device__ __align__(256) int g_align_static_scratch[PMOE_STATIC_SCRATCH_INTS];

namespace pmoe {
namespace {

constexpr size_t kStaticScratchInts = PMOE_STATIC_SCRATCH_INTS;

// Device address of the array, looked up once per device. In host code the array's name is only a
// handle for the runtime, not an address a kernel could use, hence cudaGetSymbolAddress.
int static_scratch_ptr(int **out) {
    static int *cached[64] = {nullptr};
    int dev = 0;
    PMOE_CUDA_OK(cudaGetDevice(&dev));
    PMOE_REQUIRE(dev >= 0 && dev < 64, PMOE_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    if (!cached[dev]) {
        void *p = nullptr;
        PMOE_CUDA_OK(cudaGetSymbolAddress(&p, g_align_static_scratch));
        PMOE_REQUIRE(p != nullptr, PMOE_ERR_CUDA, "moe_align_static: no device address for the scratch array");
        cached[dev] = static_cast<int *>(p);
    }
    *out = cached[dev];
    return PMOE_OK;
}

}  // namespace
}  // namespace pmoe

extern "C" size_t pmoe_moe_align_static_capacity_bytes(void) { return pmoe::kStaticScratchInts * sizeof(int); }

extern "C" int pmoe_moe_align_static(const int32_t *topk_ids, int32_t *sorted_token_ids, int32_t *expert_ids,
                                     int32_t *num_tokens_post_padded, int n, int num_experts, int block_m,
                                     int pad_to, int max_padded, int max_blocks, pmoe_stream_t stream) {
    using namespace pmoe;
    if (int rc = check_args(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, n, num_experts,
                            block_m, pad_to, max_padded, max_blocks))
        return rc;
    const Plan p = make_plan(n, num_experts);
    PMOE_REQUIRE(p.ws_ints <= kStaticScratchInts, PMOE_ERR_UNSUPPORTED,
                 "moe_align_static: n=%d with %d experts needs %zu bytes of scratch, the built-in array holds %zu; "
                 "use pmoe_moe_align_ws with caller memory instead",
                 n, num_experts, p.ws_ints * sizeof(int), kStaticScratchInts * sizeof(int));
    int *scratch = nullptr;
    if (p.ws_ints)
        if (int rc = static_scratch_ptr(&scratch)) return rc;
    // Nothing in the scratch has to start at zero: the histogram pass writes every counter of the
    // matrix before the scatter pass reads any of them.
    return launch(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, n, num_experts, block_m, pad_to,
                  max_padded, max_blocks, p, scratch, stream);
}
