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
