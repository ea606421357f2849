// C entry points around the reference's native layer, for tests and the benchmark only.
// TEST INFRASTRUCTURE: the product never links or loads this.
//
// The reference's kernels are compiled from their sources where they lie (never copied) by
// oracle/build_ref.py; this file only declares the three `pi::` launchers with the signatures of
// prime_moe/csrc/torch_interface.cpp:11-75 and turns their C++ exceptions into status codes.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <exception>

namespace pi {
void fused_moe_bf16(const __nv_bfloat16 *x, const __nv_bfloat16 *w, const __nv_bfloat16 *w2, __nv_bfloat16 *out,
                    const int32_t *sorted_token_ids, const int32_t *expert_idxs,
                    const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k, int M, int K, int N,
                    int num_experts, int sorted_num, int block_m, int block_n, int warp_n, int stages, int bpc,
                    int cpc, bool split, cudaStream_t stream);
void fused_moe_mxfp8(const __nv_fp8_e4m3 *x, const __nv_fp8_e8m0 *x_scales, const __nv_fp8_e4m3 *w,
                     const __nv_fp8_e8m0 *w_scales, const __nv_fp8_e4m3 *w2, const __nv_fp8_e8m0 *w2_scales,
                     __nv_bfloat16 *out, const int32_t *sorted_token_ids, const int32_t *expert_idxs,
                     const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k, int M, int K,
                     int N, int num_experts, int sorted_num, int block_m, int block_n, int warp_n, int stages,
                     int bpc, bool split, cudaStream_t stream);
void moe_align(const int32_t *topk_ids, int32_t *sorted_token_ids, int32_t *expert_ids,
               int32_t *num_tokens_post_padded, int n, int num_experts, int block_m, int pad_to, int max_padded,
               int max_blocks, cudaStream_t stream);
}  // namespace pi

static thread_local char g_msg[512] = "";

template <typename F>
static int guarded(F &&f) {
    try {
        f();
        return 0;
    } catch (const std::exception &e) {
        strncpy(g_msg, e.what(), sizeof(g_msg) - 1);
        return 1;
    } catch (...) {
        strncpy(g_msg, "unknown exception", sizeof(g_msg) - 1);
        return 1;
    }
}

extern "C" const char *ref_last_error(void) { return g_msg; }

extern "C" int ref_moe_align(const int32_t *topk_ids, int32_t *sorted_token_ids, int32_t *expert_ids,
                             int32_t *num_tokens_post_padded, int n, int num_experts, int block_m, int pad_to,
                             int max_padded, int max_blocks, cudaStream_t stream) {
    return guarded([&] {
        pi::moe_align(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, n, num_experts, block_m,
                      pad_to, max_padded, max_blocks, stream);
    });
}

extern "C" int ref_fused_moe_bf16(const void *x, const void *w, const void *w2, void *out,
                                  const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                  const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k, int M,
                                  int K, int N, int num_experts, int sorted_num, int block_m, int block_n, int warp_n,
                                  int stages, int bpc, int cpc, int split, cudaStream_t stream) {
    return guarded([&] {
        pi::fused_moe_bf16(static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(w),
                           static_cast<const __nv_bfloat16 *>(w2), static_cast<__nv_bfloat16 *>(out),
                           sorted_token_ids, expert_ids, num_tokens_post_padded, topk_weights, top_k, M, K, N,
                           num_experts, sorted_num, block_m, block_n, warp_n, stages, bpc, cpc, split != 0, stream);
    });
}

extern "C" int ref_fused_moe_mxfp8(const void *x, const void *x_scales, const void *w, const void *w_scales,
                                   const void *w2, const void *w2_scales, void *out,
                                   const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                   const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k, int M,
                                   int K, int N, int num_experts, int sorted_num, int block_m, int block_n,
                                   int warp_n, int stages, int bpc, int split, cudaStream_t stream) {
    return guarded([&] {
        pi::fused_moe_mxfp8(static_cast<const __nv_fp8_e4m3 *>(x), static_cast<const __nv_fp8_e8m0 *>(x_scales),
                            static_cast<const __nv_fp8_e4m3 *>(w), static_cast<const __nv_fp8_e8m0 *>(w_scales),
                            static_cast<const __nv_fp8_e4m3 *>(w2), static_cast<const __nv_fp8_e8m0 *>(w2_scales),
                            static_cast<__nv_bfloat16 *>(out), sorted_token_ids, expert_ids, num_tokens_post_padded,
                            topk_weights, top_k, M, K, N, num_experts, sorted_num, block_m, block_n, warp_n, stages,
                            bpc, split != 0, stream);
    });
}
