// TORCH_LIBRARY registration of the prime_moe operators on top of the C ABI (include/pmoe_b200.h).
//
// Schemas, argument order, defaults and tensor-level checks mirror the reference binding
// (prime_moe/csrc/torch_interface.cpp:77-110 moe_align, :112-180 fused_moe_bf16, :182-268
// fused_moe_mxfp8, schemas :271-324) so the ops are drop-in. Shape/knob checks that the reference
// performs with TORCH_CHECK are performed by the C ABI and surface here as the same c10::Error.
// Workspaces come from torch's caching allocator (stream-ordered for the current stream) and are
// handed to the `_ws` entry points, so the op itself performs no cudaMalloc.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/all.h>
#include <torch/library.h>

#include <optional>
#include <tuple>

#include "../../include/pmoe_b200.h"

namespace {

void check_status(int rc) { TORCH_CHECK(rc == PMOE_OK, pmoe_last_error()); }

torch::Tensor workspace(size_t bytes, const torch::Tensor &like) {
    // +1024 so the pointer can be rounded up to the 1024-byte alignment the kernels need
    return torch::empty({static_cast<int64_t>(bytes + 1024)},
                        torch::TensorOptions().dtype(torch::kUInt8).device(like.device()));
}
void *align1k(void *p) {
    return reinterpret_cast<void *>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}

std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> moe_align(const torch::Tensor &topk_ids,
                                                                  int64_t num_experts, int64_t block_m,
                                                                  int64_t bpc) {
    at::cuda::OptionalCUDAGuard guard{device_of(topk_ids)};   // first: the stream below must be the current one of the tensors' device
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(topk_ids.is_contiguous());
    TORCH_CHECK(topk_ids.dtype() == torch::kInt32);
    TORCH_CHECK(block_m > 0 && bpc > 0 && num_experts > 0);
    const int64_t n = topk_ids.numel();
    const int64_t pad_to = block_m * bpc;
    const int64_t max_padded = (n + num_experts * (pad_to - 1) + pad_to - 1) / pad_to * pad_to;
    const int64_t max_blocks = max_padded / block_m;
    auto opts = torch::TensorOptions().dtype(torch::kInt32).device(topk_ids.device());
    torch::Tensor sorted_token_ids = torch::empty({max_padded}, opts);
    torch::Tensor expert_ids = torch::empty({max_blocks}, opts);
    torch::Tensor num_tokens_post_padded = torch::empty({1}, opts);
    const size_t ws_bytes = pmoe_moe_align_workspace_bytes(static_cast<int>(n), static_cast<int>(num_experts));
    torch::Tensor ws;
    void *ws_ptr = nullptr;
    if (ws_bytes) {
        ws = workspace(ws_bytes, topk_ids);
        ws_ptr = align1k(ws.data_ptr());
    }
    check_status(pmoe_moe_align_ws(static_cast<const int32_t *>(topk_ids.const_data_ptr()),
                                   static_cast<int32_t *>(sorted_token_ids.data_ptr()),
                                   static_cast<int32_t *>(expert_ids.data_ptr()),
                                   static_cast<int32_t *>(num_tokens_post_padded.data_ptr()), static_cast<int>(n),
                                   static_cast<int>(num_experts), static_cast<int>(block_m),
                                   static_cast<int>(pad_to), static_cast<int>(max_padded),
                                   static_cast<int>(max_blocks), ws_ptr, ws_bytes, stream));
    return {sorted_token_ids, expert_ids, num_tokens_post_padded};
}

void fused_moe_bf16(const torch::Tensor &x, const torch::Tensor &w, const torch::Tensor &w2,
                    const torch::Tensor &sorted_token_ids, const torch::Tensor &expert_ids,
                    const torch::Tensor &num_tokens_post_padded, const torch::Tensor &topk_weights,
                    torch::Tensor &out, int64_t top_k, int64_t block_m, int64_t block_n, int64_t warp_n,
                    int64_t stages, int64_t bpc, int64_t cpc, bool split) {
    at::cuda::OptionalCUDAGuard guard{device_of(x)};   // first: the stream below must be the current one of the tensors' device
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(x.dim() == 2 && w.dim() == 3 && w2.dim() == 3);
    TORCH_CHECK(x.size(0));
    TORCH_CHECK(x.size(1) == w.size(2));
    TORCH_CHECK(w2.size(0) == w.size(0) && w2.size(1) == x.size(1) && w2.size(2) * 2 == w.size(1),
                "w2 must have shape (E, K, N/2)");
    TORCH_CHECK(out.numel() == x.numel(), "out must have shape (M, K)");
    TORCH_CHECK(topk_weights.numel() >= x.size(0) * top_k, "topk_weights must hold M*top_k values");
    TORCH_CHECK(expert_ids.numel() * block_m >= sorted_token_ids.numel(),
                "expert_ids must cover every block of sorted_token_ids");
    TORCH_CHECK(x.is_contiguous());
    TORCH_CHECK(w.is_contiguous());
    TORCH_CHECK(w2.is_contiguous());
    TORCH_CHECK(sorted_token_ids.is_contiguous());
    TORCH_CHECK(expert_ids.is_contiguous());
    TORCH_CHECK(num_tokens_post_padded.is_contiguous());
    TORCH_CHECK(topk_weights.is_contiguous());
    TORCH_CHECK(out.is_contiguous());
    TORCH_CHECK(x.dtype() == torch::kBFloat16);
    TORCH_CHECK(w.dtype() == torch::kBFloat16);
    TORCH_CHECK(w2.dtype() == torch::kBFloat16);
    TORCH_CHECK(topk_weights.dtype() == torch::kFloat32);
    TORCH_CHECK(sorted_token_ids.dtype() == torch::kInt32);
    TORCH_CHECK(expert_ids.dtype() == torch::kInt32);
    TORCH_CHECK(num_tokens_post_padded.dtype() == torch::kInt32);
    TORCH_CHECK(out.dtype() == torch::kBFloat16);
    const int M = static_cast<int>(x.size(0)), K = static_cast<int>(x.size(1));
    const int N = static_cast<int>(w.size(1)), E = static_cast<int>(w.size(0));
    const int sorted_num = static_cast<int>(sorted_token_ids.size(0));
    const size_t ws_bytes = pmoe_fused_moe_bf16_workspace_bytes(M, K, N, sorted_num, split);
    torch::Tensor ws;
    void *ws_ptr = nullptr;
    if (ws_bytes) {
        ws = workspace(ws_bytes, x);
        ws_ptr = align1k(ws.data_ptr());
    }
    check_status(pmoe_fused_moe_bf16_ws(
        x.const_data_ptr(), w.const_data_ptr(), w2.const_data_ptr(), out.data_ptr(),
        static_cast<const int32_t *>(sorted_token_ids.const_data_ptr()),
        static_cast<const int32_t *>(expert_ids.const_data_ptr()),
        static_cast<const int32_t *>(num_tokens_post_padded.const_data_ptr()),
        static_cast<const float *>(topk_weights.const_data_ptr()), static_cast<int>(top_k), M, K, N, E, sorted_num,
        static_cast<int>(block_m), static_cast<int>(block_n), static_cast<int>(warp_n), static_cast<int>(stages),
        static_cast<int>(bpc), static_cast<int>(cpc), split ? 1 : 0, ws_ptr, ws_bytes, stream));
}

void fused_moe_mxfp8(const torch::Tensor &x, const torch::Tensor &x_scales, const torch::Tensor &w,
                     const torch::Tensor &w_scales, const torch::Tensor &w2, const torch::Tensor &w2_scales,
                     const torch::Tensor &sorted_token_ids, const torch::Tensor &expert_ids,
                     const torch::Tensor &num_tokens_post_padded, const torch::Tensor &topk_weights,
                     torch::Tensor &out, int64_t top_k, int64_t block_m, int64_t block_n, int64_t warp_n,
                     int64_t stages, int64_t bpc, bool split) {
    at::cuda::OptionalCUDAGuard guard{device_of(x)};   // first: the stream below must be the current one of the tensors' device
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(x.dim() == 2 && w.dim() == 3 && w2.dim() == 3);
    const int64_t M = x.size(0), K = x.size(1), E = w.size(0), N = w.size(1);
    TORCH_CHECK(M);
    TORCH_CHECK(K == w.size(2));
    TORCH_CHECK((K & 255) == 0, "K dimension must be a multiple of 256 on the mxfp8 path");
    TORCH_CHECK((N & 255) == 0, "N dimension must be a multiple of 256 on the mxfp8 path");
    TORCH_CHECK(w2.size(0) == E && w2.size(1) == K && w2.size(2) == N / 2);
    TORCH_CHECK(x_scales.numel() == M * (K / 32), "x_scales must be a row major (M, K/32) e8m0 tensor");
    TORCH_CHECK(w_scales.numel() == E * N * (K / 32),
                "w_scales must hold E*N*K/32 e8m0 values in the blocked layout");
    TORCH_CHECK(w2_scales.numel() == E * K * ((N / 2) / 32),
                "w2_scales must hold E*K*(N/2)/32 e8m0 values in the blocked layout");
    TORCH_CHECK(out.numel() == x.numel(), "out must have shape (M, K)");
    TORCH_CHECK(topk_weights.numel() >= M * top_k, "topk_weights must hold M*top_k values");
    TORCH_CHECK(expert_ids.numel() * block_m >= sorted_token_ids.numel(),
                "expert_ids must cover every block of sorted_token_ids");
    TORCH_CHECK(x.is_contiguous());
    TORCH_CHECK(x_scales.is_contiguous());
    TORCH_CHECK(w.is_contiguous());
    TORCH_CHECK(w_scales.is_contiguous());
    TORCH_CHECK(w2.is_contiguous());
    TORCH_CHECK(w2_scales.is_contiguous());
    TORCH_CHECK(sorted_token_ids.is_contiguous());
    TORCH_CHECK(expert_ids.is_contiguous());
    TORCH_CHECK(num_tokens_post_padded.is_contiguous());
    TORCH_CHECK(topk_weights.is_contiguous());
    TORCH_CHECK(out.is_contiguous());
    TORCH_CHECK(x.dtype() == torch::kFloat8_e4m3fn);
    TORCH_CHECK(x_scales.dtype() == torch::kFloat8_e8m0fnu);
    TORCH_CHECK(w.dtype() == torch::kFloat8_e4m3fn);
    TORCH_CHECK(w_scales.dtype() == torch::kFloat8_e8m0fnu);
    TORCH_CHECK(w2.dtype() == torch::kFloat8_e4m3fn);
    TORCH_CHECK(w2_scales.dtype() == torch::kFloat8_e8m0fnu);
    TORCH_CHECK(topk_weights.dtype() == torch::kFloat32);
    TORCH_CHECK(sorted_token_ids.dtype() == torch::kInt32);
    TORCH_CHECK(expert_ids.dtype() == torch::kInt32);
    TORCH_CHECK(num_tokens_post_padded.dtype() == torch::kInt32);
    TORCH_CHECK(out.dtype() == torch::kBFloat16);
    const int sorted_num = static_cast<int>(sorted_token_ids.size(0));
    const size_t ws_bytes = pmoe_fused_moe_mxfp8_workspace_bytes(static_cast<int>(M), static_cast<int>(K),
                                                                 static_cast<int>(N), sorted_num, split);
    torch::Tensor ws;
    void *ws_ptr = nullptr;
    if (ws_bytes) {
        ws = workspace(ws_bytes, x);
        ws_ptr = align1k(ws.data_ptr());
    }
    check_status(pmoe_fused_moe_mxfp8_ws(
        x.const_data_ptr(), x_scales.const_data_ptr(), w.const_data_ptr(), w_scales.const_data_ptr(),
        w2.const_data_ptr(), w2_scales.const_data_ptr(), out.data_ptr(),
        static_cast<const int32_t *>(sorted_token_ids.const_data_ptr()),
        static_cast<const int32_t *>(expert_ids.const_data_ptr()),
        static_cast<const int32_t *>(num_tokens_post_padded.const_data_ptr()),
        static_cast<const float *>(topk_weights.const_data_ptr()), static_cast<int>(top_k), static_cast<int>(M),
        static_cast<int>(K), static_cast<int>(N), static_cast<int>(E), sorted_num, static_cast<int>(block_m),
        static_cast<int>(block_n), static_cast<int>(warp_n), static_cast<int>(stages), static_cast<int>(bpc),
        split ? 1 : 0, ws_ptr, ws_bytes, stream));
}

// expert-parallel plan (not in the reference): visits (token, destination rank) ordered by rank, see pmoe_ep_plan.
// Returns (counts[world], visit_token[Vmax], visit_meta[Vmax, 2*top_k], slot_of[T, world]), all int32;
// only the first sum(counts) visits are meaningful.
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> ep_plan(const torch::Tensor &topk_ids,
                                                                               const torch::Tensor &topk_weights,
                                                                               int64_t num_experts, int64_t world) {
    at::cuda::OptionalCUDAGuard guard{device_of(topk_ids)};   // first: the stream below must be the current one of the tensors' device
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(topk_ids.dim() == 2 && topk_ids.is_contiguous() && topk_ids.dtype() == torch::kInt32,
                "topk_ids must be a contiguous int32 [T, top_k] tensor");
    TORCH_CHECK(topk_weights.is_contiguous() && topk_weights.dtype() == torch::kFloat32 &&
                    topk_weights.numel() == topk_ids.numel(),
                "topk_weights must be contiguous fp32 with one weight per route");
    TORCH_CHECK(world > 0 && num_experts > 0);
    const int64_t T = topk_ids.size(0), top_k = topk_ids.size(1);
    const int64_t vmax = T * std::min<int64_t>(top_k, world);
    auto opts = topk_ids.options();
    torch::Tensor counts = torch::empty({world}, opts);
    torch::Tensor visit_token = torch::empty({vmax}, opts);
    torch::Tensor visit_meta = torch::empty({vmax, 2 * top_k}, opts);
    torch::Tensor slot_of = torch::empty({T, world}, opts);
    const size_t ws_bytes = pmoe_ep_plan_workspace_bytes(static_cast<int>(T), static_cast<int>(world));
    torch::Tensor ws = torch::empty({static_cast<int64_t>(ws_bytes / 4) + 1}, opts);
    check_status(pmoe_ep_plan(static_cast<const int32_t *>(topk_ids.const_data_ptr()),
                              static_cast<const float *>(topk_weights.const_data_ptr()), static_cast<int>(T),
                              static_cast<int>(top_k), static_cast<int>(num_experts), static_cast<int>(world),
                              static_cast<int32_t *>(counts.data_ptr()), static_cast<int32_t *>(visit_token.data_ptr()),
                              static_cast<int32_t *>(visit_meta.data_ptr()), static_cast<int32_t *>(slot_of.data_ptr()),
                              ws.data_ptr(), ws_bytes, stream));
    return {counts, visit_token, visit_meta, slot_of};
}

// expert-parallel combine: out[t] = sum over the token's visits of y[slot_of[t, g]] (not in the reference)
torch::Tensor ep_combine(const torch::Tensor &y, const torch::Tensor &slot_of) {
    at::cuda::OptionalCUDAGuard guard{device_of(y)};   // first: the stream below must be the current one of the tensors' device
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(y.dim() == 2 && y.is_contiguous() && y.dtype() == torch::kBFloat16);
    TORCH_CHECK(slot_of.dim() == 2 && slot_of.is_contiguous() && slot_of.dtype() == torch::kInt32);
    const int64_t T = slot_of.size(0), world = slot_of.size(1), K = y.size(1);
    torch::Tensor out = torch::empty({T, K}, y.options());
    check_status(pmoe_ep_combine(y.const_data_ptr(), static_cast<const int32_t *>(slot_of.const_data_ptr()),
                                 out.data_ptr(), static_cast<int>(T), static_cast<int>(world), static_cast<int>(K),
                                 stream));
    return out;
}

// router (not in the reference: "routing comes from your gate", README.md:147): logits [T, E] fp32 or bf16 ->
// (topk_ids int32 [T, top_k], topk_weights fp32 [T, top_k]), see pmoe_route_topk
std::tuple<torch::Tensor, torch::Tensor> route_topk(const torch::Tensor &logits, int64_t top_k, bool renormalize) {
    at::cuda::OptionalCUDAGuard guard{device_of(logits)};
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous(), "logits must be a contiguous [T, E] tensor");
    TORCH_CHECK(logits.dtype() == torch::kFloat32 || logits.dtype() == torch::kBFloat16,
                "logits must be fp32 or bf16");
    const int64_t T = logits.size(0), E = logits.size(1);
    torch::Tensor ids = torch::empty({T, top_k}, logits.options().dtype(torch::kInt32));
    torch::Tensor wts = torch::empty({T, top_k}, logits.options().dtype(torch::kFloat32));
    check_status(pmoe_route_topk(logits.const_data_ptr(),
                                 logits.dtype() == torch::kFloat32 ? PMOE_DTYPE_F32 : PMOE_DTYPE_BF16,
                                 static_cast<int>(T), static_cast<int>(E), static_cast<int>(top_k), renormalize ? 1 : 0,
                                 static_cast<int32_t *>(ids.data_ptr()), static_cast<float *>(wts.data_ptr()), stream));
    return {ids, wts};
}

// router + moe_align in one call (pmoe_route_topk_align): (topk_ids, topk_weights, sorted_token_ids, expert_ids,
// num_tokens_post_padded); the last three exactly as prime_moe::moe_align would return them for topk_ids
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> route_topk_align(
    const torch::Tensor &logits, int64_t top_k, bool renormalize, int64_t block_m, int64_t bpc) {
    at::cuda::OptionalCUDAGuard guard{device_of(logits)};
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous(), "logits must be a contiguous [T, E] tensor");
    TORCH_CHECK(logits.dtype() == torch::kFloat32 || logits.dtype() == torch::kBFloat16,
                "logits must be fp32 or bf16");
    TORCH_CHECK(block_m > 0 && bpc > 0 && top_k > 0);
    const int64_t T = logits.size(0), E = logits.size(1), n = T * top_k, pad_to = block_m * bpc;
    const int64_t max_padded = (n + E * (pad_to - 1) + pad_to - 1) / pad_to * pad_to;
    auto i32 = logits.options().dtype(torch::kInt32);
    torch::Tensor ids = torch::empty({T, top_k}, i32), wts = torch::empty({T, top_k}, logits.options().dtype(torch::kFloat32));
    torch::Tensor sorted = torch::empty({max_padded}, i32), experts = torch::empty({max_padded / block_m}, i32);
    torch::Tensor npp = torch::empty({1}, i32);
    const size_t ws_bytes = pmoe_moe_align_workspace_bytes(static_cast<int>(n), static_cast<int>(E));
    torch::Tensor ws = torch::empty({static_cast<int64_t>(ws_bytes) + 16}, logits.options().dtype(torch::kUInt8));
    check_status(pmoe_route_topk_align(
        logits.const_data_ptr(), logits.dtype() == torch::kFloat32 ? PMOE_DTYPE_F32 : PMOE_DTYPE_BF16, static_cast<int>(T),
        static_cast<int>(E), static_cast<int>(top_k), renormalize ? 1 : 0, static_cast<int32_t *>(ids.data_ptr()),
        static_cast<float *>(wts.data_ptr()), static_cast<int32_t *>(sorted.data_ptr()),
        static_cast<int32_t *>(experts.data_ptr()), static_cast<int32_t *>(npp.data_ptr()), static_cast<int>(block_m),
        static_cast<int>(pad_to), static_cast<int>(max_padded), static_cast<int>(max_padded / block_m), ws.data_ptr(),
        ws_bytes, stream));
    return {ids, wts, sorted, experts, npp};
}

// activation quantiser (not in the reference: README.md:110-113 leaves it to the caller): bf16 [T, K] ->
// (e4m3 [R, K], e8m0 [R, K/32]); with row_index int32 [R] output row r is x[row_index[r]], see pmoe_quantize_mx
std::tuple<torch::Tensor, torch::Tensor> quantize_mx(const torch::Tensor &x,
                                                     const std::optional<torch::Tensor> &row_index) {
    at::cuda::OptionalCUDAGuard guard{device_of(x)};
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.dtype() == torch::kBFloat16,
                "x must be a contiguous bf16 [T, K] tensor");
    const int64_t T = x.size(0), K = x.size(1);
    TORCH_CHECK(K % 32 == 0, "K must be a multiple of 32");
    int64_t R = T;
    const int32_t *index = nullptr;
    if (row_index.has_value()) {
        TORCH_CHECK(row_index->dtype() == torch::kInt32 && row_index->is_contiguous() && row_index->device() == x.device(),
                    "row_index must be a contiguous int32 tensor on the device of x");
        R = row_index->numel();
        index = static_cast<const int32_t *>(row_index->const_data_ptr());
    }
    torch::Tensor q = torch::empty({R, K}, x.options().dtype(torch::kFloat8_e4m3fn));
    torch::Tensor sc = torch::empty({R, K / 32}, x.options().dtype(torch::kFloat8_e8m0fnu));
    check_status(pmoe_quantize_mx(x.const_data_ptr(), index, static_cast<int>(T), q.data_ptr(), sc.data_ptr(),
                                  static_cast<int>(R), static_cast<int>(K), stream));
    return {q, sc};
}

// backward pass of fused_moe_bf16 (not in the reference, which is forward-only: README.md:17); see
// pmoe_fused_moe_bf16_backward. Returns (d_x, d_w, d_w2, d_topk_weights).
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> fused_moe_bf16_backward(
    const torch::Tensor &x, const torch::Tensor &w, const torch::Tensor &w2, const torch::Tensor &d_out,
    const torch::Tensor &sorted_token_ids, const torch::Tensor &expert_ids, const torch::Tensor &num_tokens_post_padded,
    const torch::Tensor &topk_weights, int64_t top_k, const std::optional<torch::Tensor> &gate_up) {
    at::cuda::OptionalCUDAGuard guard{device_of(x)};
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(x.dim() == 2 && w.dim() == 3 && w2.dim() == 3, "x must be [T, K], w [E, N, K], w2 [E, K, N/2]");
    const void *gu = nullptr;
    if (gate_up.has_value()) {
        TORCH_CHECK(gate_up->is_cuda() && gate_up->is_contiguous() && gate_up->dtype() == torch::kBFloat16 &&
                        gate_up->numel() == sorted_token_ids.numel() * w.size(1),
                    "gate_up must be the contiguous bf16 [sorted_num, N] tensor of fused_moe_bf16_keep");
        gu = gate_up->const_data_ptr();
    }
    for (const torch::Tensor *t : {&x, &w, &w2, &d_out})
        TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->dtype() == torch::kBFloat16,
                    "x, w, w2 and d_out must be contiguous bf16 CUDA tensors");
    for (const torch::Tensor *t : {&sorted_token_ids, &expert_ids, &num_tokens_post_padded})
        TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->dtype() == torch::kInt32,
                    "the routing tensors must be contiguous int32 CUDA tensors");
    TORCH_CHECK(topk_weights.is_cuda() && topk_weights.is_contiguous() && topk_weights.dtype() == torch::kFloat32,
                "topk_weights must be a contiguous fp32 CUDA tensor");
    const int64_t T = x.size(0), K = x.size(1), E = w.size(0), N = w.size(1);
    TORCH_CHECK(w.size(2) == K && w2.size(0) == E && w2.size(1) == K && w2.size(2) * 2 == N, "weight shapes do not match");
    TORCH_CHECK(d_out.sizes() == x.sizes(), "d_out must have the shape of x");
    TORCH_CHECK(topk_weights.numel() == T * top_k, "topk_weights must hold T * top_k entries");
    torch::Tensor d_x = torch::empty_like(x), d_w = torch::empty_like(w), d_w2 = torch::empty_like(w2);
    torch::Tensor d_wt = torch::empty({T, top_k}, topk_weights.options());
    const size_t need = pmoe_fused_moe_bf16_backward_workspace_bytes(
        static_cast<int>(T), static_cast<int>(K), static_cast<int>(N), static_cast<int>(E), static_cast<int>(top_k),
        static_cast<int>(sorted_token_ids.numel()));
    torch::Tensor ws = torch::empty({static_cast<int64_t>(need) + 1024}, x.options().dtype(torch::kUInt8));
    void *ws_ptr = reinterpret_cast<void *>((reinterpret_cast<uintptr_t>(ws.data_ptr()) + 1023) & ~static_cast<uintptr_t>(1023));
    check_status(pmoe_fused_moe_bf16_backward(
        x.const_data_ptr(), w.const_data_ptr(), w2.const_data_ptr(), d_out.const_data_ptr(),
        static_cast<const int32_t *>(sorted_token_ids.const_data_ptr()),
        static_cast<const int32_t *>(expert_ids.const_data_ptr()),
        static_cast<const int32_t *>(num_tokens_post_padded.const_data_ptr()),
        static_cast<const float *>(topk_weights.const_data_ptr()), static_cast<int>(top_k), static_cast<int>(T),
        static_cast<int>(K), static_cast<int>(N), static_cast<int>(E), static_cast<int>(sorted_token_ids.numel()),
        d_x.data_ptr(), d_w.data_ptr(), d_w2.data_ptr(), static_cast<float *>(d_wt.data_ptr()), gu, ws_ptr, need,
        stream));
    return {d_x, d_w, d_w2, d_wt};
}

// forward call that keeps the gate/up pre-activations for the backward pass (pmoe_fused_moe_bf16_keep_ws):
// writes `out`, returns gate_up bf16 [sorted_num, N]
torch::Tensor fused_moe_bf16_keep(const torch::Tensor &x, const torch::Tensor &w, const torch::Tensor &w2,
                                  const torch::Tensor &sorted_token_ids, const torch::Tensor &expert_ids,
                                  const torch::Tensor &num_tokens_post_padded, const torch::Tensor &topk_weights,
                                  torch::Tensor &out, int64_t top_k, int64_t bpc) {
    at::cuda::OptionalCUDAGuard guard{device_of(x)};
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(x.dim() == 2 && w.dim() == 3 && w2.dim() == 3, "x must be [T, K], w [E, N, K], w2 [E, K, N/2]");
    for (const torch::Tensor *t : {&x, &w, &w2, static_cast<const torch::Tensor *>(&out)})
        TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->dtype() == torch::kBFloat16,
                    "x, w, w2 and out must be contiguous bf16 CUDA tensors");
    for (const torch::Tensor *t : {&sorted_token_ids, &expert_ids, &num_tokens_post_padded})
        TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->dtype() == torch::kInt32,
                    "the routing tensors must be contiguous int32 CUDA tensors");
    TORCH_CHECK(topk_weights.is_cuda() && topk_weights.is_contiguous() && topk_weights.dtype() == torch::kFloat32,
                "topk_weights must be a contiguous fp32 CUDA tensor");
    const int64_t T = x.size(0), K = x.size(1), E = w.size(0), N = w.size(1), R = sorted_token_ids.numel();
    TORCH_CHECK(w.size(2) == K && w2.size(0) == E && w2.size(1) == K && w2.size(2) * 2 == N, "weight shapes do not match");
    TORCH_CHECK(out.sizes() == x.sizes(), "out must have the shape of x");
    torch::Tensor gate_up = torch::empty({R, N}, x.options());
    const size_t need = pmoe_fused_moe_bf16_workspace_bytes(static_cast<int>(T), static_cast<int>(K), static_cast<int>(N),
                                                            static_cast<int>(R), 1);
    torch::Tensor ws = torch::empty({static_cast<int64_t>(need) + 1024}, x.options().dtype(torch::kUInt8));
    void *ws_ptr = reinterpret_cast<void *>((reinterpret_cast<uintptr_t>(ws.data_ptr()) + 1023) & ~static_cast<uintptr_t>(1023));
    check_status(pmoe_fused_moe_bf16_keep_ws(
        x.const_data_ptr(), w.const_data_ptr(), w2.const_data_ptr(), out.data_ptr(),
        static_cast<const int32_t *>(sorted_token_ids.const_data_ptr()),
        static_cast<const int32_t *>(expert_ids.const_data_ptr()),
        static_cast<const int32_t *>(num_tokens_post_padded.const_data_ptr()),
        static_cast<const float *>(topk_weights.const_data_ptr()), static_cast<int>(top_k), static_cast<int>(T),
        static_cast<int>(K), static_cast<int>(N), static_cast<int>(E), static_cast<int>(R), static_cast<int>(bpc),
        gate_up.data_ptr(), ws_ptr, need, stream));
    return gate_up;
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(prime_moe, m) {
    m.def("fused_moe_bf16_backward(Tensor x, Tensor w, Tensor w2, Tensor d_out, Tensor sorted_token_ids, "
          "Tensor expert_ids, Tensor num_tokens_post_padded, Tensor topk_weights, int top_k, Tensor? gate_up=None) -> "
          "(Tensor, Tensor, Tensor, Tensor)");
    m.impl("fused_moe_bf16_backward", torch::kCUDA, &fused_moe_bf16_backward);
    m.def("fused_moe_bf16_keep(Tensor x, Tensor w, Tensor w2, Tensor sorted_token_ids, Tensor expert_ids, "
          "Tensor num_tokens_post_padded, Tensor topk_weights, Tensor(a!) out, int top_k, int bpc=1) -> Tensor");
    m.impl("fused_moe_bf16_keep", torch::kCUDA, &fused_moe_bf16_keep);
    m.def("route_topk(Tensor logits, int top_k, bool renormalize=True) -> (Tensor, Tensor)");
    m.impl("route_topk", torch::kCUDA, &route_topk);
    m.def("route_topk_align(Tensor logits, int top_k, bool renormalize=True, int block_m=128, int bpc=1) -> "
          "(Tensor, Tensor, Tensor, Tensor, Tensor)");
    m.impl("route_topk_align", torch::kCUDA, &route_topk_align);
    m.def("quantize_mx(Tensor x, Tensor? row_index=None) -> (Tensor, Tensor)");
    m.impl("quantize_mx", torch::kCUDA, &quantize_mx);
    m.def("ep_plan(Tensor topk_ids, Tensor topk_weights, int num_experts, int world) -> (Tensor, Tensor, Tensor, Tensor)");
    m.impl("ep_plan", torch::kCUDA, &ep_plan);
    m.def("ep_combine(Tensor y, Tensor slot_of) -> Tensor");
    m.impl("ep_combine", torch::kCUDA, &ep_combine);
    m.def(
        "fused_moe_bf16(Tensor x, Tensor w, Tensor w2, Tensor sorted_token_ids, Tensor expert_ids, "
        "Tensor num_tokens_post_padded, Tensor topk_weights, Tensor(a!) out, int top_k, int block_m, "
        "int block_n, int warp_n, int stages, int bpc, int cpc, bool split=True) -> ()");
    m.impl("fused_moe_bf16", torch::kCUDA, &fused_moe_bf16);
    m.def(
        "fused_moe_mxfp8(Tensor x, Tensor x_scales, Tensor w, Tensor w_scales, Tensor w2, Tensor w2_scales, "
        "Tensor sorted_token_ids, Tensor expert_ids, Tensor num_tokens_post_padded, Tensor topk_weights, "
        "Tensor(a!) out, int top_k, int block_m, int block_n, int warp_n, int stages, int bpc, "
        "bool split=True) -> ()");
    m.impl("fused_moe_mxfp8", torch::kCUDA, &fused_moe_mxfp8);
    m.def("moe_align(Tensor topk_ids, int num_experts, int block_m, int bpc) -> (Tensor, Tensor, Tensor)");
    m.impl("moe_align", torch::kCUDA, &moe_align);
}
