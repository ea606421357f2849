// The two steps a caller runs right before the fused MoE FFN, as HBM-bound kernels of this library:
//
//   pmoe_route_topk   router logits [T, E] -> topk_ids int32 [T, top_k], topk_weights fp32 [T, top_k]
//                     (softmax + top-k in one pass over the logits). The reference leaves routing to the
//                     caller ("routing comes from your gate", README.md:147) and only fixes the contract of
//                     the two tensors (prime_moe/csrc/torch_interface.cpp:77-110, :112-180).
//   pmoe_quantize_mx  bf16 rows -> OCP-MX operands (e4m3 values + one e8m0 scale per 32 elements), optionally
//                     gathering the rows through an index (the expert-parallel dispatch). The reference leaves
//                     this to the caller as well (README.md:110-113); the arithmetic to match bit for bit is
//                     its test quantiser (test/test_mxfp8.py:21-38): e = clamp(exponent(amax) - 8, 0, 254),
//                     q = satfinite_e4m3(v * 2^(127 - e)).
//
// Algorithmic bytes: route 4*T*E (or 2*T*E for bf16 logits) read + 8*T*top_k written;
// quantise 2*R*K read + R*K + R*K/32 written.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <algorithm>

#include "host_common.h"
#include "route_warp.cuh"

namespace pmoe {
namespace {

// ---------------------------------------------------------------------------------------------
// router: one warp per token, lane l holds logits l, l+32, ... in registers
// ---------------------------------------------------------------------------------------------
constexpr int kRouteWarps = 8;

// PER = ceil(E / 32) rounded up to a power of two (1..32): registers per lane
template <typename T, int PER>
__global__ void __launch_bounds__(kRouteWarps * 32)
route_topk_kernel(const T *__restrict__ logits, int tokens, int E, int top_k, int renormalize,
                  int32_t *__restrict__ topk_ids, float *__restrict__ topk_weights) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * kRouteWarps + (threadIdx.x >> 5);
    if (t >= tokens) return;
    int idx;
    float w;
    route_token_warp<T, PER>(logits + static_cast<size_t>(t) * E, E, top_k, renormalize, lane, idx, w);
    if (lane < top_k) {
        topk_ids[static_cast<size_t>(t) * top_k + lane] = idx;
        topk_weights[static_cast<size_t>(t) * top_k + lane] = w;
    }
}

template <typename T>
int launch_route(const T *logits, int tokens, int E, int top_k, int renormalize, int32_t *ids, float *wts,
                 cudaStream_t stream) {
    const int grid = (tokens + kRouteWarps - 1) / kRouteWarps;
    const int per = (E + 31) / 32;
#define PMOE_ROUTE_CASE(P)                                                                                         \
    if (per <= P) {                                                                                                \
        route_topk_kernel<T, P><<<grid, kRouteWarps * 32, 0, stream>>>(logits, tokens, E, top_k, renormalize, ids, \
                                                                      wts);                                        \
        PMOE_CUDA_OK(cudaGetLastError());                                                                          \
        return PMOE_OK;                                                                                            \
    }
    PMOE_ROUTE_CASE(1)
    PMOE_ROUTE_CASE(2)
    PMOE_ROUTE_CASE(4)
    PMOE_ROUTE_CASE(8)
    PMOE_ROUTE_CASE(16)
    PMOE_ROUTE_CASE(32)
#undef PMOE_ROUTE_CASE
    return set_error(PMOE_ERR_UNSUPPORTED, "route_topk supports at most 1024 experts, got %d", E);
}

// ---------------------------------------------------------------------------------------------
// MX quantiser
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

// One thread per 32-element block: four 16-byte loads (64 contiguous bytes), the block maximum, the e8m0 exponent,
// 32 e4m3 values as two 16-byte stores and one scale byte (consecutive threads, consecutive scale bytes).
__global__ void __launch_bounds__(256)
quantize_mx_kernel(const __nv_bfloat16 *__restrict__ x, const int32_t *__restrict__ row_index, int src_rows,
                   uint8_t *__restrict__ q, uint8_t *__restrict__ scales, int rows, int K) {
    const int kblocks = K / 32;
    const long long total = static_cast<long long>(rows) * kblocks;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i / kblocks), kb = static_cast<int>(i - static_cast<long long>(r) * kblocks);
        const int src = row_index ? row_index[r] : r;
        const bool live = src >= 0 && src < src_rows;       // rows with an index outside x are written as zeros
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            raw[u] = make_uint4(0, 0, 0, 0);
            if (live) raw[u] = __ldg(reinterpret_cast<const uint4 *>(x + static_cast<size_t>(src) * K + kb * 32) + u);
        }
        float v[32];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw[u]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[u * 8 + 2 * j] = __low2float(h[j]);
                v[u * 8 + 2 * j + 1] = __high2float(h[j]);
            }
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
        int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu) - 8;
        e = max(0, min(e, 254));
        const uint32_t field = static_cast<uint32_t>(254 - e);
        const float inv = __uint_as_float(field ? field << 23 : 0x00400000u);   // 2^(127-e); 2^-127 is subnormal
        uint4 o[2];
        uint32_t *ow = reinterpret_cast<uint32_t *>(o);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            ow[j] = e4m3x4(v[4 * j] * inv, v[4 * j + 1] * inv, v[4 * j + 2] * inv, v[4 * j + 3] * inv);
        uint4 *dst = reinterpret_cast<uint4 *>(q + static_cast<size_t>(r) * K + kb * 32);
        dst[0] = o[0];
        dst[1] = o[1];
        scales[i] = static_cast<uint8_t>(e);
    }
}

}  // namespace
}  // namespace pmoe

extern "C" int pmoe_route_topk(const void *logits, int logits_dtype, int T, int num_experts, int top_k,
                               int renormalize, int32_t *topk_ids, float *topk_weights, pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(logits && topk_ids && topk_weights, PMOE_ERR_BAD_ARG, "route_topk: null pointer");
    PMOE_REQUIRE(T >= 0 && num_experts > 0 && top_k > 0, PMOE_ERR_BAD_ARG,
                 "route_topk: T >= 0, num_experts > 0 and top_k > 0 required");
    PMOE_REQUIRE(top_k <= 32 && top_k <= num_experts, PMOE_ERR_UNSUPPORTED,
                 "route_topk: top_k must be at most min(32, num_experts), got %d", top_k);
    PMOE_REQUIRE(logits_dtype == PMOE_DTYPE_F32 || logits_dtype == PMOE_DTYPE_BF16, PMOE_ERR_BAD_ARG,
                 "route_topk: logits_dtype must be PMOE_DTYPE_F32 or PMOE_DTYPE_BF16");
    if (T == 0) return PMOE_OK;
    if (logits_dtype == PMOE_DTYPE_F32)
        return launch_route(static_cast<const float *>(logits), T, num_experts, top_k, renormalize ? 1 : 0, topk_ids,
                            topk_weights, stream);
    return launch_route(static_cast<const __nv_bfloat16 *>(logits), T, num_experts, top_k, renormalize ? 1 : 0,
                        topk_ids, topk_weights, stream);
}

extern "C" int pmoe_quantize_mx(const void *x, const int32_t *row_index, int src_rows, void *q, void *scales, int rows,
                                int K, pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(x && q && scales, PMOE_ERR_BAD_ARG, "quantize_mx: null pointer");
    PMOE_REQUIRE(rows >= 0 && src_rows >= 0 && K > 0 && K % 32 == 0, PMOE_ERR_BAD_ARG,
                 "quantize_mx: rows >= 0 and K a positive multiple of 32 required");
    PMOE_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q)) & 15) == 0, PMOE_ERR_BAD_ARG,
                 "quantize_mx: x and q must be 16-byte aligned");
    if (rows == 0) return PMOE_OK;
    const long long total = static_cast<long long>(rows) * (K / 32);
    const int grid = static_cast<int>(std::min<long long>((total + 255) / 256, 16ll * sm_count()));
    quantize_mx_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x), row_index, src_rows,
                                                 static_cast<uint8_t *>(q), static_cast<uint8_t *>(scales), rows, K);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}
