// moe_align for sm_100a: warp-aggregated histogram -> scan -> stable scatter.
//
// Contract (same outputs as pi::moe_align, prime_moe/csrc/kernels/fused_moe_bf16_kernel.cu:853-928):
//   sorted_token_ids[max_padded]: for every expert its pair ids followed by -1 up to a multiple of
//   pad_to, experts in ascending order, -1 after num_tokens_post_padded;
//   expert_ids[max_blocks]: expert owning each block_m-row block (largest e with offs[e] <= row),
//   num_experts-1 for blocks past the end; num_tokens_post_padded[0] = sum of padded counts.
// The reference runs ONE CTA with shared-memory atomics and a serial scan, and leaves the order
// inside an expert to the atomics. Here the ids are cut into contiguous per-warp segments; a warp
// counts its segment with __match_any_sync groups (no atomics at all, counters are private to the
// warp), a scan kernel turns the per-warp counts into per-warp write cursors, and the scatter pass
// replays the segments in order - so the result is deterministic and ascending inside each expert.
//
// HBM traffic: 2 x 4n bytes of ids read, 4*max_padded written twice at most (-1 fill + scatter),
// plus the E x (#warps) counter matrix (scratch).
#include <stdio.h>

#include "host_common.h"

namespace pmoe {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;
constexpr int kSmallN = 4096;      // up to here a single CTA does everything, no scratch
constexpr int kIdsPerWarpMin = 256;
constexpr int kMaxExperts = 1024;

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// Count the ids of [begin, end) into cnt[0..E) (private to the calling warp, already zeroed).
__device__ __forceinline__ void warp_histogram(const int32_t *__restrict__ ids, int begin, int end, int E,
                                               int *cnt) {
    const int lane = threadIdx.x & 31;
    for (int base = begin; base < end; base += 32) {
        const int i = base + lane;
        int id = (i < end) ? ids[i] : -1;
        const bool valid = id >= 0 && id < E;
        if (!valid) id = -1;
        const unsigned peers = __match_any_sync(0xffffffffu, id);
        if (valid && (peers & lanemask_lt()) == 0) cnt[id] += __popc(peers);
        __syncwarp();
    }
}

// Replay [begin, end): cur[e] is this warp's next write position for expert e.
__device__ __forceinline__ void warp_scatter(const int32_t *__restrict__ ids, int begin, int end, int E,
                                             int *cur, int32_t *__restrict__ sorted, int max_padded) {
    const int lane = threadIdx.x & 31;
    for (int base = begin; base < end; base += 32) {
        const int i = base + lane;
        int id = (i < end) ? ids[i] : -1;
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
__global__ void __launch_bounds__(kThreads) moe_align_small_kernel(
    const int32_t *__restrict__ ids, int32_t *__restrict__ sorted, int32_t *__restrict__ expert_ids,
    int32_t *__restrict__ npp, int n, int E, int block_m, int pad_to, int max_padded, int max_blocks) {
    extern __shared__ int sm[];
    int *cnt = sm;                       // [kWarpsPerCta][E]
    int *tot = cnt + kWarpsPerCta * E;   // [E]
    int *offs = tot + E;                 // [E + 1]
    int *wsum = offs + E + 1;            // [kWarpsPerCta]
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < kWarpsPerCta * E; i += kThreads) cnt[i] = 0;
    __syncthreads();
    const int seg = ((n + kWarpsPerCta - 1) / kWarpsPerCta + 31) & ~31;
    const int begin = min(warp * seg, n), end = min(begin + seg, n);
    warp_histogram(ids, begin, end, E, cnt + warp * E);
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += kThreads) {
        int run = 0;
        for (int w = 0; w < kWarpsPerCta; ++w) {
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
    for (int i = threadIdx.x; i < max_padded; i += kThreads) sorted[i] = -1;
    for (int j = threadIdx.x; j < max_blocks; j += kThreads) {
        const int row = j * block_m;
        expert_ids[j] = row >= total ? E - 1 : find_expert(offs, E, row);
    }
    for (int e = threadIdx.x; e < E; e += kThreads) {
        const int o = offs[e];
        for (int w = 0; w < kWarpsPerCta; ++w) cnt[w * E + e] += o;
    }
    __syncthreads();  // orders the -1 fill before the scatter stores of this CTA
    warp_scatter(ids, begin, end, E, cnt + warp * E, sorted, max_padded);
}

// ---------------------------------------------------------------------------------------------
// general n: histogram (grid) -> scan (1 CTA) -> scatter (grid)
//   counts is [E][num_warps] (expert-major, so the scan reads rows contiguously)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) moe_align_hist_kernel(
    const int32_t *__restrict__ ids, int n, int E, int seg, int num_warps, int *__restrict__ counts,
    int32_t *__restrict__ sorted, int max_padded) {
    extern __shared__ int sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int *cnt = sm + warp * E;
    for (int e = lane; e < E; e += 32) cnt[e] = 0;
    __syncwarp();
    const int gw = blockIdx.x * kWarpsPerCta + warp;
    const int begin = min(gw * seg, n), end = min(begin + seg, n);
    warp_histogram(ids, begin, end, E, cnt);
    for (int e = lane; e < E; e += 32) counts[static_cast<size_t>(e) * num_warps + gw] = cnt[e];
    // -1 everywhere; the scatter kernel (later in stream order) overwrites the valid slots
    int4 *s4 = reinterpret_cast<int4 *>(sorted);
    const int n4 = max_padded >> 2;
    const int4 m1 = make_int4(-1, -1, -1, -1);
    for (int i = blockIdx.x * kThreads + threadIdx.x; i < n4; i += gridDim.x * kThreads) s4[i] = m1;
    if (blockIdx.x == 0 && threadIdx.x < (max_padded & 3)) sorted[(n4 << 2) + threadIdx.x] = -1;
}

__global__ void __launch_bounds__(1024) moe_align_scan_kernel(
    int *__restrict__ counts, int num_warps, int E, int block_m, int pad_to, int *__restrict__ offs_out,
    int32_t *__restrict__ npp, int32_t *__restrict__ expert_ids, int max_blocks) {
    extern __shared__ int sm[];
    int *tot = sm;            // [E]
    int *offs = tot + E;      // [E + 1]
    int *wsum = offs + E + 1; // [32]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = warp; e < E; e += 32) {
        int *row = counts + static_cast<size_t>(e) * num_warps;
        int carry = 0;
        for (int base = 0; base < num_warps; base += 32) {
            const int idx = base + lane;
            const int v = idx < num_warps ? row[idx] : 0;
            int incl = v;
            for (int d = 1; d < 32; d <<= 1) {
                const int u = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += u;
            }
            if (idx < num_warps) row[idx] = carry + incl - v;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) tot[e] = carry;
    }
    __syncthreads();
    block_offsets(tot, offs, wsum, E, pad_to);
    const int total = offs[E];
    if (threadIdx.x == 0) npp[0] = total;
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offs_out[e] = offs[e];
    for (int j = threadIdx.x; j < max_blocks; j += blockDim.x) {
        const int row = j * block_m;
        expert_ids[j] = row >= total ? E - 1 : find_expert(offs, E, row);
    }
}

__global__ void __launch_bounds__(kThreads) moe_align_scatter_kernel(
    const int32_t *__restrict__ ids, int n, int E, int seg, int num_warps, const int *__restrict__ counts,
    const int *__restrict__ offs, int32_t *__restrict__ sorted, int max_padded) {
    extern __shared__ int sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int *cur = sm + warp * E;
    const int gw = blockIdx.x * kWarpsPerCta + warp;
    for (int e = lane; e < E; e += 32) cur[e] = counts[static_cast<size_t>(e) * num_warps + gw] + offs[e];
    __syncwarp();
    const int begin = min(gw * seg, n), end = min(begin + seg, n);
    warp_scatter(ids, begin, end, E, cur, sorted, max_padded);
}

struct Plan {
    int ctas;       // grid of the histogram / scatter kernels (0 = single-CTA path)
    int num_warps;
    int seg;        // ids per warp (multiple of 32)
    size_t ws_ints; // scratch ints
};

Plan make_plan(int n, int E) {
    Plan p{};
    if (n <= kSmallN) return p;
    int warps = (n + kIdsPerWarpMin - 1) / kIdsPerWarpMin;
    int ctas = (warps + kWarpsPerCta - 1) / kWarpsPerCta;
    const int max_ctas = 2 * sm_count();
    if (ctas > max_ctas) ctas = max_ctas;
    p.ctas = ctas;
    p.num_warps = ctas * kWarpsPerCta;
    p.seg = ((n + p.num_warps - 1) / p.num_warps + 31) & ~31;
    p.ws_ints = static_cast<size_t>(E) * p.num_warps + E + 1;
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
        const size_t smem = (static_cast<size_t>(kWarpsPerCta) * E + 2 * E + 1 + kWarpsPerCta) * sizeof(int);
        moe_align_small_kernel<<<1, kThreads, smem, stream>>>(topk_ids, sorted, expert_ids, npp, n, E, block_m,
                                                             pad_to, max_padded, max_blocks);
        PMOE_CUDA_OK(cudaGetLastError());
        return PMOE_OK;
    }
    int *counts = ws;
    int *offs = ws + static_cast<size_t>(E) * p.num_warps;
    const size_t smem_w = static_cast<size_t>(kWarpsPerCta) * E * sizeof(int);
    moe_align_hist_kernel<<<p.ctas, kThreads, smem_w, stream>>>(topk_ids, n, E, p.seg, p.num_warps, counts,
                                                                sorted, max_padded);
    PMOE_CUDA_OK(cudaGetLastError());
    const size_t smem_s = (2 * static_cast<size_t>(E) + 1 + 32) * sizeof(int);
    moe_align_scan_kernel<<<1, 1024, smem_s, stream>>>(counts, p.num_warps, E, block_m, pad_to, offs, npp,
                                                       expert_ids, max_blocks);
    PMOE_CUDA_OK(cudaGetLastError());
    moe_align_scatter_kernel<<<p.ctas, kThreads, smem_w, stream>>>(topk_ids, n, E, p.seg, p.num_warps, counts,
                                                                   offs, sorted, max_padded);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}

}  // namespace
}  // namespace pmoe

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
// For them the per-warp counter matrix and the offset table live in a fixed array that is part of
// the library image. Every GPU that loads the library carries these 4 MiB until the process exits.
#define PMOE_STATIC_SCRATCH_INTS (1u << 20)  /* 4 MiB: the stated maximum */
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
    // matrix and the scan pass writes every offset before anything reads them.
    return launch(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, n, num_experts, block_m, pad_to,
                  max_padded, max_blocks, p, scratch, stream);
}
