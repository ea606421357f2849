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

// order-preserving map float -> uint32 (larger float, larger key; -inf is the smallest key of a finite or infinite
// value) and back, so that the warp-wide maximum is ONE redux instruction
__device__ __forceinline__ uint32_t float_key(float v) {
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// PER = ceil(E / 32) rounded up to a power of two (1..32): registers per lane. On return lane j < top_k holds the
// j-th selected expert (descending logit, ties to the lower index) and its routing weight.
// Every lane caches the best of its own PER logits; a round is then two warp reductions (redux.sync: the largest
// key, and the lowest expert index among the lanes holding it) and only the winning lane rescans its registers.
template <typename T, int PER>
__device__ __forceinline__ void route_token_warp(const T *__restrict__ row, int E, int top_k, int renormalize, int lane,
                                                 int &my_idx, float &my_weight) {
    constexpr unsigned kFull = 0xffffffffu;
    float v[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? load_logit<T>(row + e) : -CUDART_INF_F;
    }
    auto local_best = [&](uint32_t &key, int &best_e) {   // lowest index among this lane's largest logits
        float best = -CUDART_INF_F;
        best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = lane + 32 * i;
            if (e < E && (v[i] > best || best_e == 0x7fffffff)) {
                best = v[i];
                best_e = e;
            }
        }
        key = float_key(best);
    };
    uint32_t lkey;
    int lbest;
    local_best(lkey, lbest);
    const float m = key_float(__reduce_max_sync(kFull, lkey));
    float sum = 0.f;
    if (!renormalize) {
#pragma unroll
        for (int i = 0; i < PER; ++i) sum += (lane + 32 * i < E) ? expf(v[i] - m) : 0.f;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(kFull, sum, d);
    }
    float my_val = 0.f;
    my_idx = 0;
    for (int j = 0; j < top_k; ++j) {
        const uint32_t kmax = __reduce_max_sync(kFull, lkey);
        const int e_win = __reduce_min_sync(kFull, lkey == kmax ? lbest : 0x7fffffff);
        if (lane == j) {
            my_val = key_float(kmax);
            my_idx = e_win;
        }
        if ((e_win & 31) == lane) {          // the owner drops the taken logit and refreshes its cached best
#pragma unroll
            for (int i = 0; i < PER; ++i)
                if (i == (e_win >> 5)) v[i] = -CUDART_INF_F;
            local_best(lkey, lbest);
        }
    }
    const float p = lane < top_k ? expf(my_val - m) : 0.f;
    if (renormalize) {
        sum = p;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(kFull, sum, d);
    }
    my_weight = p / sum;
}

}  // namespace pmoe
