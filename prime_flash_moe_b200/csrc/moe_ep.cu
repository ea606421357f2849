// Expert-parallel glue kernels (no counterpart in the reference, which is single-GPU).
//
// ep_combine: after the combine all-to-all every (token, route) pair's expert output sits in some row
// ("slot") of a [P, K] bf16 buffer; out[t, :] = bf16( sum_j w[t, j] * y[slot[t*top_k + j], :] ) with
// fp32 accumulation. One pass: top_k rows read, one row written. HBM-bound:
// P*K*2 bytes read + T*K*2 written.
#include <cuda_bf16.h>

#include <algorithm>

#include "host_common.h"

namespace pmoe {
namespace {

__global__ void __launch_bounds__(256)
ep_combine_kernel(const __nv_bfloat16 *__restrict__ y, const long long *__restrict__ slots,
                  const float *__restrict__ weights, __nv_bfloat16 *__restrict__ out, int T, int top_k, int K) {
    const int chunks = K / 8;
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < top_k; ++j) {
                const long long slot = slots[static_cast<long long>(t) * top_k + j];
                const float w = weights[static_cast<long long>(t) * top_k + j];
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(y + slot * K) + c);
                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[2 * i] += w * __low2float(h[i]);
                    acc[2 * i + 1] += w * __high2float(h[i]);
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

extern "C" int pmoe_ep_combine(const void *y, const int64_t *slot_of_pair, const float *weights, void *out, int T,
                               int top_k, int K, pmoe_stream_t stream) {
    using namespace pmoe;
    PMOE_REQUIRE(y && slot_of_pair && weights && out, PMOE_ERR_BAD_ARG, "ep_combine: null pointer");
    PMOE_REQUIRE(T >= 0 && top_k > 0 && K > 0 && K % 8 == 0, PMOE_ERR_BAD_ARG,
                 "ep_combine: T >= 0, top_k > 0 and K a positive multiple of 8 required");
    PMOE_REQUIRE(((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15) == 0, PMOE_ERR_BAD_ARG,
                 "ep_combine: y and out must be 16-byte aligned");
    if (T == 0) return PMOE_OK;
    ep_combine_kernel<<<std::min(T, 8 * sm_count()), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(y), reinterpret_cast<const long long *>(slot_of_pair), weights,
        static_cast<__nv_bfloat16 *>(out), T, top_k, K);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}
