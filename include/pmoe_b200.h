/* C ABI of the B200 (sm_100a) fused MoE FFN library `libpmoe_b200.so`.
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer unless stated otherwise, `stream`
 * is a CUDA stream handle (cudaStream_t / CUstream), and every function returns a status code
 * (PMOE_OK == 0) instead of throwing; `pmoe_last_error()` returns the message of the last failing
 * call on the calling thread. No entry point synchronises the host with the device except
 * `pmoe_device_status` and `pmoe_reset_device_status`.
 *
 * Each entry point names the reference interface it replaces (file:line inside
 * PrimeIntellect-ai/prime-flash-moe). Argument order and meaning follow the reference's native
 * `pi::` layer so that its torch binding can forward to these functions one to one.
 */
#ifndef PMOE_B200_H
#define PMOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st *pmoe_stream_t;

enum {
    PMOE_OK = 0,
    PMOE_ERR_BAD_ARG = 1,     /* an argument violates the documented contract */
    PMOE_ERR_UNSUPPORTED = 2, /* a knob combination this library (like the reference) rejects */
    PMOE_ERR_CUDA = 3,        /* a CUDA runtime / driver call failed */
    PMOE_ERR_DEVICE = 4       /* a kernel recorded an error (bounded wait expired) */
};

/* Message of the last error on this thread ("" if none). The pointer stays valid until the next
 * failing call on the same thread. */
const char *pmoe_last_error(void);

/* Library version: major * 10000 + minor * 100 + patch. */
int pmoe_version(void);

/* ---------------------------------------------------------------------------------------------
 * moe_align: counting sort of (token, route) pair ids by expert with per-expert padding.
 * Replaces pi::moe_align (prime_moe/csrc/torch_interface.cpp:63-75, kernel
 * prime_moe/csrc/kernels/fused_moe_bf16_kernel.cu:853-928).
 *
 *   topk_ids               int32[n]            expert of pair i (pair id i = token * top_k + route)
 *   sorted_token_ids       int32[max_padded]   out: per expert, its pair ids in ascending order, then
 *                                              -1 up to a multiple of pad_to; -1 past the end
 *   expert_ids             int32[max_blocks]   out: expert of each block_m-row block; num_experts-1
 *                                              for blocks past num_tokens_post_padded
 *   num_tokens_post_padded int32[1]            out: sum of the padded expert counts
 *   pad_to = block_m * bpc; max_padded = ceil((n + E*(pad_to-1)) / pad_to) * pad_to;
 *   max_blocks = max_padded / block_m (prime_moe/csrc/torch_interface.cpp:88-91).
 *
 * Unlike the reference (order inside an expert left to shared-memory atomics), the order inside an
 * expert is deterministic: ascending pair id. Ids outside [0, num_experts) are ignored.
 * num_experts <= 1024 as in the reference (fused_moe_bf16_kernel.cu:922-923).
 *
 * `pmoe_moe_align` takes its scratch from the stream-ordered allocator (cudaMallocAsync);
 * `pmoe_moe_align_ws` uses caller memory of at least `pmoe_moe_align_workspace_bytes` bytes
 * (may be 0 for small n), 16-byte aligned, and performs no allocation. */
int pmoe_moe_align(const int32_t *topk_ids, int32_t *sorted_token_ids, int32_t *expert_ids,
                   int32_t *num_tokens_post_padded, int n, int num_experts, int block_m, int pad_to,
                   int max_padded, int max_blocks, pmoe_stream_t stream);
size_t pmoe_moe_align_workspace_bytes(int n, int num_experts);
int pmoe_moe_align_ws(const int32_t *topk_ids, int32_t *sorted_token_ids, int32_t *expert_ids,
                      int32_t *num_tokens_post_padded, int n, int num_experts, int block_m, int pad_to,
                      int max_padded, int max_blocks, void *workspace, size_t workspace_bytes,
                      pmoe_stream_t stream);

/* moe_align for callers that cannot allocate device memory. This entry point has no counterpart in
 * the reference. Hosts with a device-memory budget frozen after start-up, plugins that run inside
 * another framework's allocator or stream callback, and processes whose device memory already
 * belongs to a pool they do not control cannot call cudaMalloc (nor a stream-ordered or framework
 * allocator) where routing runs, and may have no spare buffer to lend to `pmoe_moe_align_ws`.
 * Same arguments and results as `pmoe_moe_align`; the scratch (one counter per thread block and expert)
 * is a fixed 256 KiB array inside the library image, held by every GPU that loads the library until
 * the process exits. The call performs no cudaMalloc, cudaFree or any other allocating routine.
 *  - Limit: inputs whose scratch need (`pmoe_moe_align_workspace_bytes(n, num_experts)`) exceeds
 *    `pmoe_moe_align_static_capacity_bytes()` are rejected with PMOE_ERR_UNSUPPORTED and a message
 *    naming both sizes; nothing is launched. n <= 4096 needs no scratch at all.
 *  - The first call on each device looks up the array's device address (with that device current);
 *    make that first call outside of any stream capture.
 *  - All calls on a device share the one array, which keeps the previous call's contents. The kernels
 *    write every counter and offset before reading it, so nothing needs clearing; but two calls that
 *    overlap on the GPU (different streams, or graph branches) race on it - serialise them. */
int pmoe_moe_align_static(const int32_t *topk_ids, int32_t *sorted_token_ids, int32_t *expert_ids,
                          int32_t *num_tokens_post_padded, int n, int num_experts, int block_m, int pad_to,
                          int max_padded, int max_blocks, pmoe_stream_t stream);
size_t pmoe_moe_align_static_capacity_bytes(void);

/* ---------------------------------------------------------------------------------------------
 * fused_moe_bf16: out[token] (+)= sum over routes  w_route * (SwiGLU(x[token] * W1[e]^T) * W2[e]^T)
 * Replaces pi::fused_moe_bf16 (prime_moe/csrc/torch_interface.cpp:11-34; kernels
 * prime_moe/csrc/kernels/fused_moe_bf16_kernel.cu:21-373, 393-546; launcher :549-733, :930-964).
 *
 *   x   bf16[M, K]        w   bf16[E, N, K]  (rows [0,N/2) gate, [N/2,N) up)     w2  bf16[E, K, N/2]
 *   out bf16[M, K]        sorted_token_ids int32[sorted_num], expert_ids int32[>= sorted_num/128],
 *   num_tokens_post_padded int32[1], topk_weights fp32[M*top_k] (indexed by pair id)
 *   block_m == 128; (block_n, warp_n) in {(32,8), (64,4)}; stages 1..5 (<= 4 when split);
 *   bpc in {1, 2} (2 = two-CTA MMA; needs moe_align run with the same bpc); cpc == 1;
 *   K % 128 == 0, N % 256 == 0.
 *   split == 0: one GEMM launch (gate/up + down per tile, split-K partials reduced in an fp32 workspace
 *               buffer) followed by a small launch that ADDS the rounded sums to `out` (caller zeroes it).
 *   split != 0: gate/up kernel -> activation workspace -> down kernel chained by programmatic
 *               dependent launch; `out` is zeroed by the library.
 * `_ws` variant: caller-provided workspace (>= pmoe_fused_moe_bf16_workspace_bytes, 1024-byte
 * aligned), no allocation; the plain variant uses cudaMallocAsync / cudaFreeAsync on `stream`. */
int pmoe_fused_moe_bf16(const void *x, const void *w, const void *w2, void *out,
                        const int32_t *sorted_token_ids, const int32_t *expert_ids,
                        const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k, int M,
                        int K, int N, int num_experts, int sorted_num, int block_m, int block_n, int warp_n,
                        int stages, int bpc, int cpc, int split, pmoe_stream_t stream);
size_t pmoe_fused_moe_bf16_workspace_bytes(int M, int K, int N, int sorted_num, int split);
/* `_ex`: the `_ws` call with two optional device-side extras (no counterpart in the reference; NULL = off):
 *   live_rows  int32[1]: only the first *live_rows rows of x / out are in use (a buffer sized for the worst case
 *              of an expert-parallel step): the library zeroes only those rows of `out`;
 *   out_rows   uint64[M] (bf16, split only): row i of the output lives at address out_rows[i], which may be another
 *              GPU's memory mapped into this process; results are ADDED there with plain vector reductions and
 *              nothing is zeroed by the library (`out` itself is then unused but must still be a valid pointer). */
int pmoe_fused_moe_bf16_ex(const void *x, const void *w, const void *w2, void *out, const int32_t *sorted_token_ids,
                           const int32_t *expert_ids, const int32_t *num_tokens_post_padded,
                           const float *topk_weights, int top_k, int M, int K, int N, int num_experts, int sorted_num,
                           int block_m, int block_n, int warp_n, int stages, int bpc, int cpc, int split,
                           void *workspace, size_t workspace_bytes, const int32_t *live_rows,
                           const unsigned long long *out_rows, pmoe_stream_t stream);
int pmoe_fused_moe_bf16_ws(const void *x, const void *w, const void *w2, void *out,
                           const int32_t *sorted_token_ids, const int32_t *expert_ids,
                           const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k,
                           int M, int K, int N, int num_experts, int sorted_num, int block_m, int block_n,
                           int warp_n, int stages, int bpc, int cpc, int split, void *workspace,
                           size_t workspace_bytes, pmoe_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * fused_moe_mxfp8: the same contraction on OCP-MX operands (e4m3 values, one e8m0 scale per 32
 * K-elements); the SwiGLU output is re-quantised to mxfp8 on chip before the down projection.
 * Replaces pi::fused_moe_mxfp8 (prime_moe/csrc/torch_interface.cpp:36-61; kernels
 * prime_moe/csrc/kernels/fused_moe_mxfp8_kernel.cu:82-503, 513-679; launcher :681-866, :944-1009).
 *
 *   x e4m3[M, K], x_scales e8m0[M, K/32] row major;
 *   w e4m3[E, N, K], w_scales e8m0[E*N*K/32] in the blocked layout of pack_scales_blocked
 *   (prime_moe/__init__.py:106-115): 512-byte tiles of 128 rows x 4 scale columns, tile index
 *   row_tile * (K/128) + k_tile, byte (r%32)*16 + (r/32)*4 + (kb%4);
 *   w2 e4m3[E, K, N/2], w2_scales e8m0[E*K*(N/2)/32] blocked likewise; K % 256 == 0, N % 256 == 0,
 *   stages 1..4; bpc in {1, 2}: 2 = CTA pairs (two-CTA block-scaled MMA; the reference's mxfp8 path rejects it),
 *   split only, needs moe_align run with bpc = 2 and 16-byte aligned packed scales. Other arguments as for bf16. */
int pmoe_fused_moe_mxfp8(const void *x, const void *x_scales, const void *w, const void *w_scales,
                         const void *w2, const void *w2_scales, void *out, const int32_t *sorted_token_ids,
                         const int32_t *expert_ids, const int32_t *num_tokens_post_padded,
                         const float *topk_weights, int top_k, int M, int K, int N, int num_experts,
                         int sorted_num, int block_m, int block_n, int warp_n, int stages, int bpc, int split,
                         pmoe_stream_t stream);
size_t pmoe_fused_moe_mxfp8_workspace_bytes(int M, int K, int N, int sorted_num, int split);
int pmoe_fused_moe_mxfp8_ex(const void *x, const void *x_scales, const void *w, const void *w_scales, const void *w2,
                            const void *w2_scales, void *out, const int32_t *sorted_token_ids,
                            const int32_t *expert_ids, const int32_t *num_tokens_post_padded,
                            const float *topk_weights, int top_k, int M, int K, int N, int num_experts, int sorted_num,
                            int block_m, int block_n, int warp_n, int stages, int bpc, int split, void *workspace,
                            size_t workspace_bytes, const int32_t *live_rows /* as for bf16 */, pmoe_stream_t stream);
int pmoe_fused_moe_mxfp8_ws(const void *x, const void *x_scales, const void *w, const void *w_scales,
                            const void *w2, const void *w2_scales, void *out,
                            const int32_t *sorted_token_ids, const int32_t *expert_ids,
                            const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k,
                            int M, int K, int N, int num_experts, int sorted_num, int block_m, int block_n,
                            int warp_n, int stages, int bpc, int split, void *workspace,
                            size_t workspace_bytes, pmoe_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * The two steps that precede the fused MoE FFN in a model. Neither has a counterpart in the reference, which
 * leaves both to the caller: routing ("routing comes from your gate", README.md:147; the op contract for the two
 * tensors is prime_moe/csrc/torch_interface.cpp:77-110, :112-180) and activation quantisation (README.md:110-113;
 * the arithmetic matched bit for bit is the reference's test quantiser, test/test_mxfp8.py:21-38).
 *
 * pmoe_route_topk: router logits [T, num_experts] (fp32 or bf16, row major) -> topk_ids int32[T, top_k] and
 *   topk_weights fp32[T, top_k], one pass over the logits. Experts are listed by descending logit; equal logits
 *   go to the lower expert index. renormalize != 0: weights = softmax over the top_k selected logits (they sum
 *   to 1, the convention of the benchmark configurations); renormalize == 0: the selected entries of the softmax
 *   over all experts. top_k <= min(32, num_experts), num_experts <= 1024.
 *
 * pmoe_quantize_mx: bf16 rows -> OCP-MX: q e4m3[rows, K] and scales e8m0[rows, K/32] (row major, one scale per
 *   32 elements: e = clamp(exponent(amax) - 8, 0, 254), q = satfinite_e4m3(v * 2^(127 - e))), the layout
 *   pmoe_fused_moe_mxfp8 takes as x / x_scales. row_index == NULL: output row r is x[r] (rows <= src_rows).
 *   row_index int32[rows]: output row r is x[row_index[r]] - the expert-parallel dispatch gather and the
 *   quantiser in one pass; an index outside [0, src_rows) yields a row of zeros. K % 32 == 0; x and q 16-byte
 *   aligned. */
enum { PMOE_DTYPE_F32 = 0, PMOE_DTYPE_BF16 = 1 };
int pmoe_route_topk(const void *logits, int logits_dtype, int T, int num_experts, int top_k, int renormalize,
                    int32_t *topk_ids, float *topk_weights, pmoe_stream_t stream);
/* Router and moe_align in one call: as pmoe_route_topk followed by pmoe_moe_align_ws on its topk_ids (same outputs,
 * bit for bit), but for n = T * top_k above the single-CTA sizes ONE kernel routes the tokens, counts its own ids
 * per expert and pre-fills sorted_token_ids - the ids are not read back for counting and one launch disappears.
 * workspace: pmoe_moe_align_workspace_bytes(T * top_k, num_experts) bytes. When top_k does not divide the id range
 * of a thread block (it does for every power of two up to 256) the two separate kernels run. */
int pmoe_route_topk_align(const void *logits, int logits_dtype, int T, int num_experts, int top_k, int renormalize,
                          int32_t *topk_ids, float *topk_weights, int32_t *sorted_token_ids, int32_t *expert_ids,
                          int32_t *num_tokens_post_padded, int block_m, int pad_to, int max_padded, int max_blocks,
                          void *workspace, size_t workspace_bytes, pmoe_stream_t stream);
int pmoe_quantize_mx(const void *x /* bf16[src_rows, K] */, const int32_t *row_index, int src_rows, void *q,
                     void *scales, int rows, int K, pmoe_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Backward pass of pmoe_fused_moe_bf16 (no counterpart in the reference, which is forward-only, README.md:17).
 * Same routing tensors as the forward call (moe_align output with block_m = 128; bpc 1 or 2 - 128-row blocks without
 * any routed row, which bpc = 2 tables contain, are skipped) and the same x,
 * w1 [E, N, K], w2 [E, K, N/2]; d_out bf16[T, K] is the gradient of `out`. Writes (does not accumulate into)
 *   d_x  bf16[T, K]        d_w1 bf16[E, N, K]        d_w2 bf16[E, K, N/2]   (experts without rows get zeros)
 *   d_topk_weights fp32[T, top_k], or NULL to skip it (entries of routes to ids outside [0, E) stay 0)
 * The gate/up pre-activations are recomputed from x unless `gate_up` is given (see below); products accumulate
 * in fp32 and every intermediate is rounded to bf16 once. K % 64 == 0, N % 128 == 0, sorted_num % 128 == 0,
 * tensors 16-byte aligned (d_w1, d_w2: 32), workspace 1024-byte aligned with pmoe_fused_moe_bf16_backward_workspace_bytes() bytes.
 * Asynchronous on `stream`; bounded waits and status reporting as for the forward kernels. */
size_t pmoe_fused_moe_bf16_backward_workspace_bytes(int T, int K, int N, int num_experts, int top_k, int sorted_num);
int pmoe_fused_moe_bf16_backward(const void *x, const void *w1, const void *w2, const void *d_out,
                                 const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                 const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k, int T,
                                 int K, int N, int num_experts, int sorted_num, void *d_x, void *d_w1, void *d_w2,
                                 float *d_topk_weights, const void *gate_up, void *workspace,
                                 size_t workspace_bytes, pmoe_stream_t stream);
/* The same with a choice of how the weight gradients are delivered: dw_dtype PMOE_DTYPE_BF16 or PMOE_DTYPE_F32 (d_w1,
 * d_w2 are then fp32 tensors of the same shapes), accumulate_dw != 0 adds to what d_w1 / d_w2 hold instead of
 * overwriting it (a trainer's fp32 main gradients over several micro-batches: the read-modify-write happens in the
 * weight-gradient kernel's epilogue, every element owned by one thread, no atomics, and the separate bf16 gradient
 * tensor with its add pass disappears). Experts without rows are left alone when accumulating. */
int pmoe_fused_moe_bf16_backward_ex(const void *x, const void *w1, const void *w2, const void *d_out,
                                    const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                    const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k, int T,
                                    int K, int N, int num_experts, int sorted_num, void *d_x, void *d_w1, void *d_w2,
                                    float *d_topk_weights, const void *gate_up, int dw_dtype, int accumulate_dw,
                                    void *workspace, size_t workspace_bytes, pmoe_stream_t stream);
/* Forward call that keeps what the backward pass would otherwise recompute: pmoe_fused_moe_bf16_ws with the knobs
 * fixed (block_m 128, split pipeline; bpc 1 or 2 as moe_align was run) whose gate/up kernel also stores its pre-activations (bf16, as rounded
 * from the fp32 accumulators) into gate_up bf16[sorted_num, N] (32-byte aligned; row r = row r of sorted_token_ids,
 * columns [0, N/2) gate, [N/2, N) up; rows of padding hold values nobody uses, 128-row blocks without any routed
 * row may stay unwritten). Passing that buffer as
 * `gate_up` to pmoe_fused_moe_bf16_backward skips its recompute GEMM (a quarter of the step on wide layers); NULL
 * there means recompute. No counterpart in the reference. */
int pmoe_fused_moe_bf16_keep_ws(const void *x, const void *w, const void *w2, void *out,
                                const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k, int M,
                                int K, int N, int num_experts, int sorted_num, int bpc, void *gate_up,
                                void *workspace, size_t workspace_bytes, pmoe_stream_t stream);
/* Measurement hook: which steps of the backward pass run. Bits: 1 row maps + row gathers, 2 gate/up recompute,
 * 4 d_act + SwiGLU derivative, 8 d_w2, 16 d_xs, 32 d_w1, 64 d_x combine; 127 = all (default). Returns the old mask.
 * With bits missing the outputs are incomplete. */
int pmoe_debug_set_backward_mask(int mask);

/* ---------------------------------------------------------------------------------------------
 * Expert-parallel glue (no counterpart in the reference, which is single-GPU). Experts are sharded
 * contiguously over `world` ranks (num_experts / world each). The unit of exchange is a VISIT: a (token,
 * destination rank) pair such that at least one of the token's top_k experts lives on that rank.
 *
 * pmoe_ep_plan: from this rank's topk_ids int32[T, top_k] and topk_weights fp32[T, top_k] writes
 *   counts int32[world]           visits per destination rank; V = their sum (<= T * min(top_k, world))
 *   visit_token int32[V]          token of each visit; visits ordered by destination rank, tokens ascending
 *   visit_meta int32[V, 2*top_k]  per visit: top_k local expert ids (-1 where the route goes elsewhere), then
 *                                 the top_k routing weights as fp32 bit patterns (0 where it goes elsewhere)
 *   slot_of int32[T, world]       visit index of (token, rank), -1 if the token does not visit that rank
 * The arrays are sized by the caller for the upper bound of V. Ids outside [0, num_experts) are ignored.
 * workspace: pmoe_ep_plan_workspace_bytes(T, world) bytes, 4-byte aligned. world <= 32.
 *
 * pmoe_ep_combine: after the return exchange, y bf16[V, K] holds one row per visit (the weighted partial sum
 * over the visited rank's experts); out[t, :] = bf16(sum over g with slot_of[t, g] >= 0 of y[slot_of[t, g], :]),
 * fp32 accumulation. K % 8 == 0; y and out 16-byte aligned. */
size_t pmoe_ep_plan_workspace_bytes(int T, int world);
int pmoe_ep_plan(const int32_t *topk_ids, const float *topk_weights, int T, int top_k, int num_experts, int world,
                 int32_t *counts, int32_t *visit_token, int32_t *visit_meta, int32_t *slot_of, void *workspace,
                 size_t workspace_bytes, pmoe_stream_t stream);
int pmoe_ep_combine(const void *y, const int32_t *slot_of, void *out, int T, int world, int K, pmoe_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Expert-parallel exchange over peer memory: the dispatch and the combine of a step as kernels of this library
 * that store straight into the other ranks' buffers over NVLink - no NCCL call and no host synchronisation
 * inside a step. No counterpart in the reference (single GPU). One process per GPU.
 *
 * Every rank allocates ONE buffer of the same size with pmoe_ep_buffer_alloc (cudaMalloc, zero-filled; the
 * 64-byte handle goes to the other ranks by any host channel), maps its peers' buffers with
 * pmoe_ep_buffer_open, and keeps the G base pointers (its own at index `rank`) in a DEVICE array `peer_bufs`.
 * A buffer starts with a header of pmoe_ep_header_bytes() bytes that the peers write (per-phase step flags and
 * the G x G matrix of visit counts); behind it, at offsets the caller chooses identically on all ranks (16-byte
 * aligned): the row area [row_cap, row_bytes], the auxiliary row area [row_cap, aux_bytes] (MX scales; aux_bytes
 * may be 0), the meta area int32[row_cap, 2*top_k] and the return area bf16[ret_cap, K]. row_cap = G * T and
 * ret_cap = T * min(top_k, G) always suffice (T = tokens per rank, the same on all ranks).
 * One step, all calls on one stream, `epoch` = 1, 2, 3, ... identical on all ranks:
 *   pmoe_ep_plan -> pmoe_ep_publish_counts -> pmoe_ep_push_rows -> pmoe_ep_recv_prepare ->
 *   pmoe_moe_align(local_ids, n = row_cap * top_k) + pmoe_fused_moe_* on x = the row area, M = row_cap,
 *   topk_weights = local_weights, out = y[row_cap, K] -> pmoe_ep_push_back -> pmoe_ep_combine_peer.
 * push_rows waits until every rank has published its counts, recv_prepare until every rank's rows have arrived
 * (then local_ids[row_cap, top_k] / local_weights hold the routing of the rows that arrived, -1 / 0 beyond, and
 * num_rows[0] their number), combine_peer until every rank has returned its partial sums; out[t] is then the
 * fp32 sum of the token's visit rows. All waits are bounded like the GEMM kernels' (pmoe_device_status codes
 * 10-12); after an expired wait the step's result is invalid. Only plain loads / stores and release / acquire
 * flag accesses touch peer memory (no TMA, no multicast, no library kernel). A rank may start step e+1 as soon
 * as its own step e has been enqueued: it writes into a peer only after that peer has returned step e. */
size_t pmoe_ep_header_bytes(void);
int pmoe_ep_buffer_alloc(size_t bytes, void **ptr, void *ipc_handle /* host, 64 bytes out */);
int pmoe_ep_buffer_open(const void *ipc_handle /* host, 64 bytes */, void **ptr);
int pmoe_ep_buffer_close(void *ptr);
int pmoe_ep_buffer_free(void *ptr);
int pmoe_ep_publish_counts(const int32_t *counts, void *const *peer_bufs, int rank, int world, int epoch,
                           pmoe_stream_t stream);
int pmoe_ep_push_rows(const void *x, int row_bytes, const void *aux, int aux_bytes, const int32_t *visit_token,
                      const int32_t *visit_meta, int top_k, int T, void *const *peer_bufs, size_t rows_off,
                      size_t aux_off, size_t meta_off, int row_cap, int rank, int world, int epoch,
                      pmoe_stream_t stream);
int pmoe_ep_recv_prepare(const void *local_buf, size_t meta_off, int top_k, int row_cap, int32_t *local_ids,
                         float *local_weights, int32_t *num_rows, int rank, int world, int epoch,
                         pmoe_stream_t stream);
int pmoe_ep_push_back(const void *y, int K, void *const *peer_bufs, size_t y_off, int row_cap, int ret_cap, int rank,
                      int world, int epoch, pmoe_stream_t stream);
/* Direct return: out_rows[i] = address of received row i's slot in the return area of the rank it came from (0
 * beyond the rows that arrived). Passed to pmoe_fused_moe_bf16_ex, the down kernels add their results straight
 * into the source ranks' return areas (vector reductions over NVLink, overlapped with the GEMM) and
 * pmoe_ep_push_back is called with y == NULL (it then only signals). The owner of a return area zeroes it
 * (cudaMemsetAsync) before its pmoe_ep_publish_counts of the step. Call after pmoe_ep_recv_prepare. */
int pmoe_ep_return_table(void *const *peer_bufs, size_t y_off, int K, int row_cap, int ret_cap, int rank, int world,
                         unsigned long long *out_rows, pmoe_stream_t stream);
int pmoe_ep_combine_peer(const void *local_buf, size_t y_off, const int32_t *slot_of, void *out, int T, int world,
                         int K, int epoch, pmoe_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Device status. Every wait inside the kernels is bounded; a wait that expires records a code in a
 * device status word and the kernel unwinds. These two calls synchronise the current device.
 * No counterpart in the reference (its waits are unbounded, tcgen05_prelude.cuh:404-414).
 *   pmoe_device_status: *status = first recorded code (0 = none); returns PMOE_OK, or
 *   PMOE_ERR_DEVICE when *status != 0.   pmoe_reset_device_status: clears the word.
 * The word is STICKY: once a code is recorded, every later kernel on that device gives up any wait that needs
 * more than a few polls, so its `out` is incomplete although the call returned PMOE_OK. Nothing but these two
 * calls reads the word (the launch path never synchronises): a host that wants to detect an expired wait calls
 * pmoe_device_status at a point where a synchronisation is acceptable (end of a step), treats every result
 * produced since the previous check as invalid when it is non-zero, and calls pmoe_reset_device_status before
 * going on. */
int pmoe_device_status(int *status /* host pointer */);
int pmoe_reset_device_status(void);

/* Profiling hook, process-wide, not thread-safe: restrict the split pipelines to a subset of their
 * launches so that each kernel can be timed alone with CUDA events (1 = row gather, 2 = gate/up
 * kernel, 4 = down kernel; default 7 = all; + 8 = without the single-block tail launches of the bpc = 2 pipeline). A partial run leaves `out` undefined. Returns the
 * previous mask. No counterpart in the reference. */
int pmoe_debug_set_phase_mask(int mask);

/* Tuning hook, process-wide: the GEMM producers prefetch weight tiles `ksteps` k-steps ahead of their
 * shared-memory ring into L2 (0 = off, the default; initial value from PMOE_L2_AHEAD). Returns the
 * previous value. No counterpart in the reference. */
int pmoe_debug_set_l2_ahead(int ksteps);

/* Test hooks for the bounded waits, per device (the current one). No counterpart in the reference.
 *   pmoe_debug_set_wait_ns: limit of every in-kernel wait in nanoseconds (default 2 s; 1 us .. 60 s).
 *   pmoe_debug_wait_probe: launches a one-CTA kernel that waits on a barrier nothing arrives on; after the
 *   current limit it records status 9 and ends through its normal exit, so pmoe_device_status then reports
 *   PMOE_ERR_DEVICE until pmoe_reset_device_status. It touches no GEMM kernel and no user memory. */
int pmoe_debug_set_wait_ns(unsigned long long ns);
int pmoe_debug_wait_probe(pmoe_stream_t stream);

/* Test hook: the number of workspace bytes the bf16 launcher would touch for this problem under the current
 * environment (PMOE_PREGATHER, PMOE_AGATHER, PMOE_PAIR_TAILS); never more than
 * pmoe_fused_moe_bf16_workspace_bytes of the same problem. Host only, no device work. */
size_t pmoe_debug_bf16_workspace_extent(int M, int K, int N, int num_experts, int top_k, int sorted_num, int bpc,
                                        int split);

#ifdef __cplusplus
}
#endif
#endif /* PMOE_B200_H */
