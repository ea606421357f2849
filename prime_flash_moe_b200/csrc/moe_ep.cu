// Expert-parallel glue kernels (no counterpart in the reference, which is single-GPU).
//
// Unit of exchange = a VISIT: one (token, destination rank) pair such that at least one of the token's
// top_k experts lives on that rank. A token row travels once per visited rank together with top_k slots of
// (local expert id or -1, routing weight or 0); the receiving rank runs the fused MoE FFN on the visits
// with those slots as its routing table, so it returns ONE row per visit - the weighted partial sum over
// its own experts - and the source adds the partial sums of a token's visits.
//
// ep_plan: visits ordered by destination rank, tokens ascending inside a rank (deterministic):
//   kernel 1  per CTA of 256 tokens: number of visits per rank            -> block_counts[rank][cta]
//   kernel 2  one CTA: exclusive scan of block_counts in (rank, cta) order -> block_base, counts[rank]
//   kernel 3  per token: visit index = block_base + rank of the token inside its CTA (ballots), then the
//             visit's token, slots and the token's slot table are written
// ep_combine: out[t, :] = bf16( sum over the token's visits of y[visit, :] ), fp32 accumulation; one pass,
//   HBM-bound: V*K*2 bytes read + T*K*2 written.
#include <cuda_bf16.h>
#include <string.h>

#include <algorithm>

#include "host_common.h"

namespace pmoe {
namespace {

constexpr int kPlanThreads = 256;
constexpr int kMaxRanks = 32;

// bit g set when one of the token's experts lives on rank g
__device__ __forceinline__ uint32_t visit_mask(const int32_t *ids, int top_k, int per_rank, int world) {
    uint32_t m = 0;
    for (int j = 0; j < top_k; ++j) {
        const int e = ids[j];
        if (e >= 0 && e < per_rank * world) m |= 1u << (e / per_rank);
    }
    return m;
}

__global__ void __launch_bounds__(kPlanThreads)
ep_plan_count_kernel(const int32_t *__restrict__ topk_ids, int T, int top_k, int per_rank, int world,
                     int32_t *__restrict__ block_counts) {
    __shared__ int s_cnt[kMaxRanks];
    if (threadIdx.x < kMaxRanks) s_cnt[threadIdx.x] = 0;
    __syncthreads();
    const int t = blockIdx.x * kPlanThreads + threadIdx.x;
    const uint32_t m = t < T ? visit_mask(topk_ids + static_cast<size_t>(t) * top_k, top_k, per_rank, world) : 0u;
    for (int g = 0; g < world; ++g) {
        const uint32_t b = __ballot_sync(0xffffffffu, (m >> g) & 1u);
        if ((threadIdx.x & 31) == 0 && b) atomicAdd(&s_cnt[g], __popc(b));
    }
    __syncthreads();
    if (threadIdx.x < world) block_counts[threadIdx.x * gridDim.x + blockIdx.x] = s_cnt[threadIdx.x];
}

// exclusive scan of n = world * blocks counts (rank-major); counts[g] = visits to rank g
__global__ void __launch_bounds__(1024)
ep_plan_scan_kernel(const int32_t *__restrict__ block_counts, int32_t *__restrict__ block_base,
                    int32_t *__restrict__ counts, int world, int blocks) {
    __shared__ int s_part[1024];
    const int n = world * blocks;
    const int per = (n + 1023) / 1024;
    const int lo = min(n, static_cast<int>(threadIdx.x) * per), hi = min(n, lo + per);
    int sum = 0;
    for (int i = lo; i < hi; ++i) sum += block_counts[i];
    s_part[threadIdx.x] = sum;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {   // Hillis-Steele inclusive scan of the 1024 partial sums
        const int v = threadIdx.x >= d ? s_part[threadIdx.x - d] : 0;
        __syncthreads();
        s_part[threadIdx.x] += v;
        __syncthreads();
    }
    int run = s_part[threadIdx.x] - sum;
    for (int i = lo; i < hi; ++i) {
        block_base[i] = run;
        run += block_counts[i];
    }
    __syncthreads();   // this CTA's block_base writes are visible to all its threads
    if (threadIdx.x < world) {
        const int start = block_base[threadIdx.x * blocks];
        const int end = static_cast<int>(threadIdx.x) + 1 < world ? block_base[(threadIdx.x + 1) * blocks] : s_part[1023];
        counts[threadIdx.x] = end - start;
    }
}

__global__ void __launch_bounds__(kPlanThreads)
ep_plan_fill_kernel(const int32_t *__restrict__ topk_ids, const float *__restrict__ topk_weights, int T, int top_k,
                    int per_rank, int world, const int32_t *__restrict__ block_base,
                    int32_t *__restrict__ visit_token, int32_t *__restrict__ visit_meta,
                    int32_t *__restrict__ slot_of) {
    __shared__ int s_warp[kPlanThreads / 32][kMaxRanks];   // visits per warp and rank
    const int t = blockIdx.x * kPlanThreads + threadIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int32_t *ids = topk_ids + static_cast<size_t>(t) * top_k;
    const uint32_t m = t < T ? visit_mask(ids, top_k, per_rank, world) : 0u;
    int rank_in_warp[kMaxRanks];
#pragma unroll 1
    for (int g = 0; g < world; ++g) {
        const uint32_t b = __ballot_sync(0xffffffffu, (m >> g) & 1u);
        if (lane == 0) s_warp[warp][g] = __popc(b);
        rank_in_warp[g] = __popc(b & ((1u << lane) - 1u));
    }
    __syncthreads();
    if (t >= T) return;
#pragma unroll 1
    for (int g = 0; g < world; ++g) {
        int v = -1;
        if ((m >> g) & 1u) {
            v = block_base[g * gridDim.x + blockIdx.x] + rank_in_warp[g];
            for (int w = 0; w < warp; ++w) v += s_warp[w][g];
            visit_token[v] = t;
            int32_t *meta = visit_meta + static_cast<size_t>(v) * 2 * top_k;
            for (int j = 0; j < top_k; ++j) {
                const int e = ids[j];
                const bool here = e >= 0 && e / per_rank == g && e < per_rank * world;
                meta[j] = here ? e - g * per_rank : -1;
                meta[top_k + j] = here ? __float_as_int(topk_weights[static_cast<size_t>(t) * top_k + j]) : 0;
            }
        }
        slot_of[static_cast<size_t>(t) * world + g] = v;
    }
}

__global__ void __launch_bounds__(256)
ep_combine_kernel(const __nv_bfloat16 *__restrict__ y, const int32_t *__restrict__ slot_of,
                  __nv_bfloat16 *__restrict__ out, int T, int world, int K) {
    const int chunks = K / 8;
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int g = 0; g < world; ++g) {
                const int slot = slot_of[static_cast<long long>(t) * world + g];
                if (slot < 0) continue;
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(y + static_cast<long long>(slot) * K) + c);
                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[2 * i] += __low2float(h[i]);
                    acc[2 * i + 1] += __high2float(h[i]);
                }
            }
            uint4 r;
            __nv_bfloat162 *o = reinterpret_cast<__nv_bfloat162 *>(&r);
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            reinterpret_cast<uint4 *>(out + static_cast<long long>(t) * K)[c] = r;
        }
    }
}

}  // namespace
}  // namespace pmoe

extern "C" size_t pmoe_ep_plan_workspace_bytes(int T, int world) {
    if (T <= 0 || world <= 0) return 0;
    const size_t blocks = (static_cast<size_t>(T) + pmoe::kPlanThreads - 1) / pmoe::kPlanThreads;
    return 2 * blocks * world * sizeof(int32_t);
}

extern "C" int pmoe_ep_plan(const int32_t *topk_ids, const float *topk_weights, int T, int top_k, int num_experts,
                            int world, int32_t *counts, int32_t *visit_token, int32_t *visit_meta, int32_t *slot_of,
                            void *workspace, size_t workspace_bytes, pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(topk_ids && topk_weights && counts && visit_token && visit_meta && slot_of, PMOE_ERR_BAD_ARG,
                 "ep_plan: null pointer");
    PMOE_REQUIRE(T >= 0 && top_k > 0 && num_experts > 0 && world > 0 && world <= kMaxRanks, PMOE_ERR_BAD_ARG,
                 "ep_plan: T >= 0, top_k > 0, num_experts > 0 and 1 <= world <= %d required", kMaxRanks);
    PMOE_REQUIRE(num_experts % world == 0, PMOE_ERR_BAD_ARG, "ep_plan: experts must divide evenly over the ranks");
    PMOE_CUDA_OK(cudaMemsetAsync(counts, 0, world * sizeof(int32_t), stream));
    if (T == 0) return PMOE_OK;
    const int blocks = (T + kPlanThreads - 1) / kPlanThreads;
    PMOE_REQUIRE(workspace && workspace_bytes >= pmoe_ep_plan_workspace_bytes(T, world), PMOE_ERR_BAD_ARG,
                 "ep_plan: workspace of %zu bytes required", pmoe_ep_plan_workspace_bytes(T, world));
    int32_t *block_counts = static_cast<int32_t *>(workspace);
    int32_t *block_base = block_counts + static_cast<size_t>(blocks) * world;
    const int per_rank = num_experts / world;
    ep_plan_count_kernel<<<blocks, kPlanThreads, 0, stream>>>(topk_ids, T, top_k, per_rank, world, block_counts);
    PMOE_CUDA_OK(cudaGetLastError());
    ep_plan_scan_kernel<<<1, 1024, 0, stream>>>(block_counts, block_base, counts, world, blocks);
    PMOE_CUDA_OK(cudaGetLastError());
    ep_plan_fill_kernel<<<blocks, kPlanThreads, 0, stream>>>(topk_ids, topk_weights, T, top_k, per_rank, world,
                                                             block_base, visit_token, visit_meta, slot_of);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}

extern "C" int pmoe_ep_combine(const void *y, const int32_t *slot_of, void *out, int T, int world, int K,
                               pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(y && slot_of && out, PMOE_ERR_BAD_ARG, "ep_combine: null pointer");
    PMOE_REQUIRE(T >= 0 && world > 0 && K > 0 && K % 8 == 0, PMOE_ERR_BAD_ARG,
                 "ep_combine: T >= 0, world > 0 and K a positive multiple of 8 required");
    PMOE_REQUIRE(((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15) == 0, PMOE_ERR_BAD_ARG,
                 "ep_combine: y and out must be 16-byte aligned");
    if (T == 0) return PMOE_OK;
    ep_combine_kernel<<<std::min(T, 8 * sm_count()), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(y), slot_of, static_cast<__nv_bfloat16 *>(out), T, world, K);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}

// =============================================================================================
// Device-driven exchange over peer memory (no NCCL call, no host synchronisation in a step)
//
// Every rank owns ONE buffer of identical layout (allocated by pmoe_ep_buffer_alloc, mapped into the peers
// through CUDA IPC). It starts with a header the PEERS write into,
//     int32 cnt_flag[32] | disp_flag[32] | comb_flag[32] | M[32][32]
// (M[s][g] = number of visits rank s sends to rank g in the current step; flag[s] = the last step for which
// rank s has finished the corresponding phase), followed at caller-chosen offsets by the row area (token rows
// received), an optional auxiliary row area (their MX scales), the meta area (top_k local expert ids + top_k
// routing weights per received row) and the return area (one bf16 row per visit this rank SENT).
// One step on rank `me`, all on one stream, step number `epoch` (1, 2, ...):
//   publish   my counts row -> M[me][.] of every rank, then cnt_flag[me] = epoch on every rank
//   push      wait until cnt_flag[s] >= epoch for all s (now M is complete and identical everywhere); visit v to
//             rank g is the j-th of my visits to g -> row  sum_{s<me} M[s][g] + j  of g's row / aux / meta areas
//             (plain 16-byte stores to peer memory); then disp_flag[me] = epoch on every rank
//   prepare   wait for disp_flag[s] >= epoch for all s; R = sum_s M[s][me] rows arrived; split the meta area into
//             the id table (rows >= R masked with -1) and the weight table for moe_align / the fused kernels
//   (moe_align + fused MoE FFN on the local experts -> y[R, K])
//   return    row i (the j-th row from source s) -> return area of s at  sum_{g<me} M[s][g] + j ; comb_flag[me] =
//             epoch on every rank
//   combine   wait for comb_flag[g] >= epoch for all g; out[t] = sum of the token's visit rows (fp32)
// A rank writes into a peer's areas for step e+1 only after its own combine of step e, which waited for that
// peer's return of step e - and the peer returns only after it has consumed the rows, meta and counts of step
// e. So one set of areas is enough. Only plain loads / stores and release / acquire flag accesses touch peer
// memory: no TMA, no multicast, no library kernel. Every wait is bounded (status word, pmoe_device_status).
// =============================================================================================
namespace pmoe {

__device__ int g_status_ep = 0;
__device__ unsigned long long g_ep_wait_ns = 2000000000ull;

namespace {

constexpr int kHdrFlagInts = 32;
constexpr int kHdrInts = 3 * kHdrFlagInts + kMaxRanks * kMaxRanks;
constexpr int ST_TIMEOUT_EP_COUNTS = 10, ST_TIMEOUT_EP_DISPATCH = 11, ST_TIMEOUT_EP_RETURN = 12;

struct Header {
    int32_t cnt_flag[kHdrFlagInts], disp_flag[kHdrFlagInts], comb_flag[kHdrFlagInts];
    int32_t M[kMaxRanks][kMaxRanks];
};
static_assert(sizeof(Header) == kHdrInts * 4, "header layout");

__device__ __forceinline__ int ld_acquire_sys(const int32_t *p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int32_t *p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// counts written by the peers: read past L1
__device__ __forceinline__ int ld_count(const int32_t *p) { return *reinterpret_cast<const volatile int32_t *>(p); }
__device__ __forceinline__ unsigned long long timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Threads 0..world-1 of the CTA wait until flag[s] >= epoch; every thread then continues. Returns false
// (after recording `code`) when the limit ran out - the caller goes on with whatever has arrived, so that the
// kernel still ends; the step's result is then invalid and the status word says so.
__device__ bool wait_flags(const int32_t *flag, int world, int epoch, int code) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < world) {
        const unsigned long long limit = *reinterpret_cast<volatile unsigned long long *>(&g_ep_wait_ns);
        const unsigned long long t0 = timer_ns();
        unsigned n = 0;
        while (ld_acquire_sys(flag + threadIdx.x) - epoch < 0) {
            if ((++n & 63u) == 0) {
                if (*reinterpret_cast<volatile int *>(&g_status_ep) != 0 || timer_ns() - t0 > limit) {
                    atomicCAS(&g_status_ep, 0, code);
                    s_ok = 0;
                    break;
                }
            }
        }
    }
    __syncthreads();
    return s_ok != 0;
}

__global__ void __launch_bounds__(32)
ep_publish_counts_kernel(const int32_t *__restrict__ counts, void *const *__restrict__ peers, int me, int world,
                         int epoch) {
    const int p = threadIdx.x;
    if (p >= world) return;
    Header *h = static_cast<Header *>(peers[p]);
    for (int g = 0; g < world; ++g) h->M[me][g] = counts[g];
    __threadfence_system();
    st_release_sys(&h->cnt_flag[me], epoch);
}

// which: 1 = disp_flag, 2 = comb_flag. Runs after the kernel whose stores it announces (stream order).
__global__ void __launch_bounds__(32)
ep_signal_kernel(void *const *__restrict__ peers, int me, int world, int epoch, int which) {
    const int p = threadIdx.x;
    if (p >= world) return;
    Header *h = static_cast<Header *>(peers[p]);
    __threadfence_system();
    st_release_sys(which == 1 ? &h->disp_flag[me] : &h->comb_flag[me], epoch);
}

struct PushArgs {
    const uint8_t *x;            // [T, row_bytes]
    const uint8_t *aux;          // [T, aux_bytes] or null
    const int32_t *visit_token;  // [V]
    const int32_t *visit_meta;   // [V, meta_ints]
    void *const *peers;
    size_t rows_off, aux_off, meta_off;
    int row_bytes, aux_bytes, meta_ints, T, me, world, epoch, row_cap;
};

__global__ void __launch_bounds__(256)
ep_push_rows_kernel(const PushArgs a) {
    __shared__ int s_send_base[kMaxRanks + 1];   // first visit of mine to rank g
    __shared__ int s_dst_base[kMaxRanks];        // first row of mine in rank g's areas
    __shared__ int s_most;                       // largest number of visits to one rank
    const Header *h = static_cast<const Header *>(a.peers[a.me]);
    wait_flags(h->cnt_flag, a.world, a.epoch, ST_TIMEOUT_EP_COUNTS);
    if (threadIdx.x == 0) {
        int run = 0;
        for (int g = 0; g < a.world; ++g) {
            s_send_base[g] = run;
            run += ld_count(&h->M[a.me][g]);
            int before = 0;
            for (int s = 0; s < a.me; ++s) before += ld_count(&h->M[s][g]);
            s_dst_base[g] = before;
        }
        s_send_base[a.world] = run;
        int most = 0;
        for (int g = 0; g < a.world; ++g) most = max(most, s_send_base[g + 1] - s_send_base[g]);
        s_most = min(most, a.T);
    }
    __syncthreads();
    // Consecutive warps serve DIFFERENT destination ranks (the j-th visit to rank me+1, me+2, ... in turn), so every
    // rank drives all its links at once and no destination is written by all ranks at the same moment; walking the
    // visits in their stored order (all of rank 0's first) made every rank hit the same peer's ingress link together.
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const long long slots = static_cast<long long>(s_most) * a.world;
    for (long long u = blockIdx.x * warps + (threadIdx.x >> 5); u < slots; u += static_cast<long long>(gridDim.x) * warps) {
        const int j = static_cast<int>(u / a.world);
        const int g = (static_cast<int>(u % a.world) + a.me + 1) % a.world;
        if (j >= s_send_base[g + 1] - s_send_base[g]) continue;
        const int v = s_send_base[g] + j;
        const long long row = static_cast<long long>(s_dst_base[g]) + j;
        if (row >= a.row_cap) continue;            // cannot happen with a row_cap of world * T; never write past an area
        const int tok = a.visit_token[v];
        if (tok < 0 || tok >= a.T) continue;
        uint8_t *base = static_cast<uint8_t *>(a.peers[g]);
        const int4 *src = reinterpret_cast<const int4 *>(a.x + static_cast<size_t>(tok) * a.row_bytes);
        int4 *dst = reinterpret_cast<int4 *>(base + a.rows_off + static_cast<size_t>(row) * a.row_bytes);
        for (int c = lane; c < a.row_bytes / 16; c += 32) dst[c] = __ldg(src + c);
        if (a.aux) {
            const int32_t *asrc = reinterpret_cast<const int32_t *>(a.aux + static_cast<size_t>(tok) * a.aux_bytes);
            int32_t *adst = reinterpret_cast<int32_t *>(base + a.aux_off + static_cast<size_t>(row) * a.aux_bytes);
            for (int c = lane; c < a.aux_bytes / 4; c += 32) adst[c] = __ldg(asrc + c);
        }
        const int32_t *msrc = a.visit_meta + static_cast<size_t>(v) * a.meta_ints;
        int32_t *mdst = reinterpret_cast<int32_t *>(base + a.meta_off) + static_cast<size_t>(row) * a.meta_ints;
        for (int c = lane; c < a.meta_ints; c += 32) mdst[c] = msrc[c];
    }
}

// ids[i, j] = local expert id of slot j of received row i (-1 for rows that did not arrive), wts[i, j] its
// routing weight; num_rows[0] = rows that arrived.
__global__ void __launch_bounds__(256)
ep_recv_prepare_kernel(const void *local_buf, size_t meta_off, int top_k, int row_cap, int32_t *__restrict__ ids,
                       float *__restrict__ wts, int32_t *__restrict__ num_rows, int me, int world, int epoch) {
    const Header *h = static_cast<const Header *>(local_buf);
    wait_flags(h->disp_flag, world, epoch, ST_TIMEOUT_EP_DISPATCH);
    int R = 0;
    for (int s = 0; s < world; ++s) R += ld_count(&h->M[s][me]);
    R = min(R, row_cap);
    if (blockIdx.x == 0 && threadIdx.x == 0) num_rows[0] = R;
    const int32_t *meta = reinterpret_cast<const int32_t *>(static_cast<const uint8_t *>(local_buf) + meta_off);
    const long long total = static_cast<long long>(row_cap) * top_k;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(i / top_k), j = static_cast<int>(i - static_cast<long long>(row) * top_k);
        const bool live = row < R;
        ids[i] = live ? __ldcg(meta + static_cast<size_t>(row) * 2 * top_k + j) : -1;
        wts[i] = live ? __int_as_float(__ldcg(meta + static_cast<size_t>(row) * 2 * top_k + top_k + j)) : 0.f;
    }
}

__global__ void __launch_bounds__(256)
ep_push_back_kernel(const __nv_bfloat16 *__restrict__ y, int K, void *const *__restrict__ peers, size_t y_off, int me,
                    int world, int row_cap, int ret_cap) {
    __shared__ int s_recv_base[kMaxRanks + 1];   // first local row that came from rank s
    __shared__ int s_ret_base[kMaxRanks];        // first visit of rank s that went to me (index in s's return area)
    __shared__ int s_most_rows;                  // largest number of rows from one rank
    const Header *h = static_cast<const Header *>(peers[me]);
    if (threadIdx.x == 0) {
        int run = 0;
        for (int s = 0; s < world; ++s) {
            s_recv_base[s] = run;
            run += ld_count(&h->M[s][me]);
            int before = 0;
            for (int g = 0; g < me; ++g) before += ld_count(&h->M[s][g]);
            s_ret_base[s] = before;
        }
        s_recv_base[world] = run;
        int most = 0;
        for (int s = 0; s < world; ++s) most = max(most, s_recv_base[s + 1] - s_recv_base[s]);
        s_most_rows = most;
    }
    __syncthreads();
    // consecutive warps return rows to different source ranks (me+1, me+2, ... in turn), as in ep_push_rows_kernel
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const long long slots = static_cast<long long>(s_most_rows) * world;
    for (long long u = blockIdx.x * warps + (threadIdx.x >> 5); u < slots; u += static_cast<long long>(gridDim.x) * warps) {
        const int j = static_cast<int>(u / world);
        const int s = (static_cast<int>(u % world) + me + 1) % world;
        if (j >= s_recv_base[s + 1] - s_recv_base[s]) continue;
        const int i = s_recv_base[s] + j;
        if (i >= row_cap) continue;
        const long long v = static_cast<long long>(s_ret_base[s]) + j;
        if (v >= ret_cap) continue;
        const int4 *src = reinterpret_cast<const int4 *>(y + static_cast<size_t>(i) * K);
        int4 *dst = reinterpret_cast<int4 *>(static_cast<uint8_t *>(peers[s]) + y_off) + static_cast<size_t>(v) * (K / 8);
        for (int c = lane; c < K / 8; c += 32) dst[c] = src[c];
    }
}

// out_rows[i] = address, in the memory of the rank row i came from, of that visit's row of the return area (0 for
// rows that did not arrive): with this table the down kernels add their results straight into the source ranks'
// buffers and no separate return pass is needed. Runs after ep_recv_prepare (the counts are complete then).
__global__ void __launch_bounds__(256)
ep_return_table_kernel(void *const *__restrict__ peers, size_t y_off, int K, int me, int world, int row_cap, int ret_cap,
                       unsigned long long *__restrict__ out_rows) {
    __shared__ int s_recv_base[kMaxRanks + 1];
    __shared__ int s_ret_base[kMaxRanks];
    const Header *h = static_cast<const Header *>(peers[me]);
    if (threadIdx.x == 0) {
        int run = 0;
        for (int s = 0; s < world; ++s) {
            s_recv_base[s] = run;
            run += ld_count(&h->M[s][me]);
            int before = 0;
            for (int g = 0; g < me; ++g) before += ld_count(&h->M[s][g]);
            s_ret_base[s] = before;
        }
        s_recv_base[world] = run;
    }
    __syncthreads();
    const int R = min(s_recv_base[world], row_cap);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < row_cap; i += gridDim.x * blockDim.x) {
        unsigned long long addr = 0;
        if (i < R) {
            int s = 0;
            while (s + 1 < world && s_recv_base[s + 1] <= i) ++s;
            const long long v = static_cast<long long>(s_ret_base[s]) + (i - s_recv_base[s]);
            if (v < ret_cap)
                addr = reinterpret_cast<unsigned long long>(static_cast<uint8_t *>(peers[s]) + y_off) +
                       static_cast<unsigned long long>(v) * K * 2ull;
        }
        out_rows[i] = addr;
    }
}

__global__ void __launch_bounds__(256)
ep_combine_peer_kernel(const void *local_buf, size_t y_off, const int32_t *__restrict__ slot_of,
                       __nv_bfloat16 *__restrict__ out, int T, int world, int K, int epoch) {
    const Header *h = static_cast<const Header *>(local_buf);
    wait_flags(h->comb_flag, world, epoch, ST_TIMEOUT_EP_RETURN);
    const __nv_bfloat16 *y = reinterpret_cast<const __nv_bfloat16 *>(static_cast<const uint8_t *>(local_buf) + y_off);
    const int chunks = K / 8;
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int g = 0; g < world; ++g) {
                const int slot = slot_of[static_cast<long long>(t) * world + g];
                if (slot < 0) continue;
                // written by a peer during this step: bypass L1 (no stale line from an earlier step)
                const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(y + static_cast<long long>(slot) * K) + c);
                const __nv_bfloat162 *hh = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[2 * i] += __low2float(hh[i]);
                    acc[2 * i + 1] += __high2float(hh[i]);
                }
            }
            uint4 r;
            __nv_bfloat162 *o = reinterpret_cast<__nv_bfloat162 *>(&r);
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            reinterpret_cast<uint4 *>(out + static_cast<long long>(t) * K)[c] = r;
        }
    }
}

int check_world(int me, int world, const char *what) {
    PMOE_REQUIRE(world >= 1 && world <= kMaxRanks && me >= 0 && me < world, PMOE_ERR_BAD_ARG,
                 "%s: 0 <= rank < world <= %d required", what, kMaxRanks);
    return PMOE_OK;
}

}  // namespace

int status_fetch_ep(int *value, bool reset) {
    if (value) PMOE_CUDA_OK(cudaMemcpyFromSymbol(value, g_status_ep, sizeof(int)));
    if (reset) {
        const int zero = 0;
        PMOE_CUDA_OK(cudaMemcpyToSymbol(g_status_ep, &zero, sizeof(int)));
    }
    return PMOE_OK;
}
int wait_ns_store_ep(unsigned long long ns) {
    PMOE_CUDA_OK(cudaMemcpyToSymbol(g_ep_wait_ns, &ns, sizeof(ns)));
    return PMOE_OK;
}

}  // namespace pmoe

extern "C" size_t pmoe_ep_header_bytes(void) { return 8192; }   // sizeof(Header) rounded up; areas start behind it

extern "C" int pmoe_ep_buffer_alloc(size_t bytes, void **ptr, void *ipc_handle) {
    using namespace pmoe;
    PMOE_REQUIRE(ptr && ipc_handle && bytes >= pmoe_ep_header_bytes(), PMOE_ERR_BAD_ARG,
                 "ep_buffer_alloc: null pointer or a buffer smaller than its header");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void *p = nullptr;
    PMOE_CUDA_OK(cudaMalloc(&p, bytes));
    PMOE_CUDA_OK(cudaMemset(p, 0, bytes));
    PMOE_CUDA_OK(cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    PMOE_CUDA_OK(cudaIpcGetMemHandle(&h, p));
    memcpy(ipc_handle, &h, sizeof(h));
    *ptr = p;
    return PMOE_OK;
}

extern "C" int pmoe_ep_buffer_open(const void *ipc_handle, void **ptr) {
    using namespace pmoe;
    PMOE_REQUIRE(ptr && ipc_handle, PMOE_ERR_BAD_ARG, "ep_buffer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle, sizeof(h));
    PMOE_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return PMOE_OK;
}

extern "C" int pmoe_ep_buffer_close(void *ptr) {
    using namespace pmoe;
    PMOE_CUDA_OK(cudaIpcCloseMemHandle(ptr));
    return PMOE_OK;
}

extern "C" int pmoe_ep_buffer_free(void *ptr) {
    using namespace pmoe;
    PMOE_CUDA_OK(cudaFree(ptr));
    return PMOE_OK;
}

extern "C" int pmoe_ep_publish_counts(const int32_t *counts, void *const *peer_bufs, int rank, int world, int epoch,
                                      pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(counts && peer_bufs, PMOE_ERR_BAD_ARG, "ep_publish_counts: null pointer");
    if (int rc = check_world(rank, world, "ep_publish_counts")) return rc;
    ep_publish_counts_kernel<<<1, 32, 0, stream>>>(counts, peer_bufs, rank, world, epoch);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}

extern "C" int pmoe_ep_push_rows(const void *x, int row_bytes, const void *aux, int aux_bytes,
                                 const int32_t *visit_token, const int32_t *visit_meta, int top_k, int T,
                                 void *const *peer_bufs, size_t rows_off, size_t aux_off, size_t meta_off, int row_cap,
                                 int rank, int world, int epoch, pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(x && visit_token && visit_meta && peer_bufs, PMOE_ERR_BAD_ARG, "ep_push_rows: null pointer");
    if (int rc = check_world(rank, world, "ep_push_rows")) return rc;
    PMOE_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && aux_bytes >= 0 && aux_bytes % 4 == 0 && top_k > 0 && T >= 0,
                 PMOE_ERR_BAD_ARG, "ep_push_rows: rows must be multiples of 16 bytes, auxiliary rows of 4 bytes");
    PMOE_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(aux) | rows_off | aux_off | meta_off) & 15) == 0,
                 PMOE_ERR_BAD_ARG, "ep_push_rows: x, aux and the area offsets must be 16-byte aligned");
    PushArgs a{static_cast<const uint8_t *>(x), aux_bytes ? static_cast<const uint8_t *>(aux) : nullptr, visit_token,
               visit_meta, peer_bufs, rows_off, aux_off, meta_off, row_bytes, aux_bytes, 2 * top_k, T, rank, world, epoch,
               row_cap};
    const int grid = std::max(1, std::min(8 * sm_count(), (T * std::min(top_k, world) + 7) / 8));
    ep_push_rows_kernel<<<grid, 256, 0, stream>>>(a);
    PMOE_CUDA_OK(cudaGetLastError());
    ep_signal_kernel<<<1, 32, 0, stream>>>(peer_bufs, rank, world, epoch, 1);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}

extern "C" int pmoe_ep_recv_prepare(const void *local_buf, size_t meta_off, int top_k, int row_cap, int32_t *local_ids,
                                    float *local_weights, int32_t *num_rows, int rank, int world, int epoch,
                                    pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(local_buf && local_ids && local_weights && num_rows, PMOE_ERR_BAD_ARG, "ep_recv_prepare: null pointer");
    if (int rc = check_world(rank, world, "ep_recv_prepare")) return rc;
    PMOE_REQUIRE(top_k > 0 && row_cap > 0, PMOE_ERR_BAD_ARG, "ep_recv_prepare: top_k and row_cap must be positive");
    const long long total = static_cast<long long>(row_cap) * top_k;
    const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>(4 * sm_count(), (total + 255) / 256)));
    ep_recv_prepare_kernel<<<grid, 256, 0, stream>>>(local_buf, meta_off, top_k, row_cap, local_ids, local_weights, num_rows,
                                                     rank, world, epoch);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}

extern "C" int pmoe_ep_push_back(const void *y, int K, void *const *peer_bufs, size_t y_off, int row_cap, int ret_cap,
                                 int rank, int world, int epoch, pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(peer_bufs, PMOE_ERR_BAD_ARG, "ep_push_back: null pointer");
    if (int rc = check_world(rank, world, "ep_push_back")) return rc;
    PMOE_REQUIRE(K > 0 && K % 8 == 0 && ((reinterpret_cast<uintptr_t>(y) | y_off) & 15) == 0, PMOE_ERR_BAD_ARG,
                 "ep_push_back: K must be a multiple of 8, y and the return area 16-byte aligned");
    if (y) {   // y == NULL: the partial sums are already in the peers' return areas (pmoe_ep_return_table): signal only
        const int grid = std::max(1, std::min(8 * sm_count(), (row_cap + 7) / 8));
        ep_push_back_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(y), K, peer_bufs, y_off, rank,
                                                      world, row_cap, ret_cap);
        PMOE_CUDA_OK(cudaGetLastError());
    }
    ep_signal_kernel<<<1, 32, 0, stream>>>(peer_bufs, rank, world, epoch, 2);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}

extern "C" int pmoe_ep_combine_peer(const void *local_buf, size_t y_off, const int32_t *slot_of, void *out, int T,
                                    int world, int K, int epoch, pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(local_buf && slot_of && out, PMOE_ERR_BAD_ARG, "ep_combine_peer: null pointer");
    PMOE_REQUIRE(T >= 0 && world > 0 && world <= kMaxRanks && K > 0 && K % 8 == 0, PMOE_ERR_BAD_ARG,
                 "ep_combine_peer: T >= 0, 1 <= world <= %d and K a positive multiple of 8 required", kMaxRanks);
    PMOE_REQUIRE(((reinterpret_cast<uintptr_t>(out) | y_off) & 15) == 0, PMOE_ERR_BAD_ARG,
                 "ep_combine_peer: out and the return area must be 16-byte aligned");
    ep_combine_peer_kernel<<<std::max(1, std::min(T, 8 * sm_count())), 256, 0, stream>>>(
        local_buf, y_off, slot_of, static_cast<__nv_bfloat16 *>(out), T, world, K, epoch);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}

extern "C" int pmoe_ep_return_table(void *const *peer_bufs, size_t y_off, int K, int row_cap, int ret_cap, int rank,
                                    int world, unsigned long long *out_rows, pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(peer_bufs && out_rows, PMOE_ERR_BAD_ARG, "ep_return_table: null pointer");
    if (int rc = check_world(rank, world, "ep_return_table")) return rc;
    PMOE_REQUIRE(K > 0 && K % 8 == 0 && (y_off & 15) == 0 && row_cap > 0, PMOE_ERR_BAD_ARG,
                 "ep_return_table: K must be a multiple of 8 and the return area 16-byte aligned");
    ep_return_table_kernel<<<std::max(1, std::min(2 * sm_count(), (row_cap + 255) / 256)), 256, 0, stream>>>(
        peer_bufs, y_off, K, rank, world, row_cap, ret_cap, out_rows);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}
