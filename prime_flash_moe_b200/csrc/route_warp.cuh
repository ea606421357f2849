// One warp routes one token: softmax + top-k over E router logits held in registers (lane l holds logits l, l+32,
// ...). Shared by the stand-alone router kernel and by the router fused with the moe_align histogram pass.
#pragma once

#include <cuda_bf16.h>
#include <math_constants.h>
#include <stdint.h>

namespace pmoe {

template <typename T>
__device__ __forceinline__ float load_logit(const T *p);
template <>
__device__ __forceinline__ float load_logit<float>(const float *p) { return __ldg(p); }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16 *p) {
    return __bfloat162float(*p);
}

// PER = ceil(E / 32) rounded up to a power of two (1..32): registers per lane. On return lane j < top_k holds the
// j-th selected expert (descending logit, ties to the lower index) and its routing weight.
template <typename T, int PER>
__device__ __forceinline__ void route_token_warp(const T *__restrict__ row, int E, int top_k, int renormalize, int lane,
                                                 int &my_idx, float &my_weight) {
    float v[PER];
    float m = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? load_logit<T>(row + e) : -CUDART_INF_F;
        m = fmaxf(m, v[i]);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    float sum = 0.f;
    if (!renormalize) {
#pragma unroll
        for (int i = 0; i < PER; ++i) sum += (lane + 32 * i < E) ? expf(v[i] - m) : 0.f;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    }
    // top_k rounds of arg-max; ties go to the lower expert index; taken entries drop to -inf
    float my_val = 0.f;
    my_idx = 0;
    for (int j = 0; j < top_k; ++j) {
        float best = -CUDART_INF_F;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = lane + 32 * i;
            if (e < E && (v[i] > best || (v[i] == best && e < best_e))) {
                best = v[i];
                best_e = e;
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, d);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, d);
            if (ob > best || (ob == best && oe < best_e)) {
                best = ob;
                best_e = oe;
            }
        }
        if (lane == j) {
            my_val = best;
            my_idx = best_e;
        }
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (lane + 32 * i == best_e) v[i] = -CUDART_INF_F;
    }
    const float p = lane < top_k ? expf(my_val - m) : 0.f;
    if (renormalize) {
        sum = p;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    }
    my_weight = p / sum;
}

}  // namespace pmoe
