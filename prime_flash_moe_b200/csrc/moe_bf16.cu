// bf16 fused MoE FFN for sm_100a: persistent, warp-specialised tcgen05 kernels.
//
// Replaces the kernels and launcher of prime_moe/csrc/kernels/fused_moe_bf16_kernel.cu
// (fused_moe_kernel :21-373, gather_x_kernel :375-391, fused_moe_down_kernel :393-546,
// launch_fused_moe_kernel_impl :549-733) behind pmoe_fused_moe_bf16.
//
// Work decomposition (all kernels): the rows of `sorted_token_ids` are cut into 128-row blocks, one
// expert per block (moe_align guarantees it). A tile is one row block x one slice of output columns.
// Each kernel is PERSISTENT: grid = min(#tiles, #SMs) CTAs, every CTA walks tiles blockIdx.x,
// blockIdx.x + gridDim.x, ...; tiles are ordered so that the up-to-8 row blocks sharing a weight
// slice run at the same time and the slice is read from HBM once and from L2 afterwards.
//
// Warp roles in every kernel:
//   warp 0        TMA producer  - fills a ring of `stages` shared-memory slots (A tile 128x64 bf16 +
//                                 B tile 256x64 bf16, 128-byte swizzle, 48 KB per slot)
//   warp 1        MMA issuer    - one thread issues tcgen05.mma (M128 x N256 x K16) into TMEM and
//                                 commits ring slots / accumulators to mbarriers; owns TMEM alloc
//   warps 2..     epilogue      - 4 or 8 warps (`warp_n`) read accumulators from TMEM
// TMEM holds 512 fp32 columns = two 128x256 accumulators, so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
//   up kernel   (split):  A = x rows gathered by token id with TMA gather4 (no gather pre-pass),
//                         B = [gate rows ; up rows] of w1[e]; epilogue: SwiGLU from TMEM -> bf16 ->
//                         swizzled staging tile -> TMA store into the activation workspace
//                         [sorted_num, H]. The 2H-wide gate/up tensor never exists in memory.
//                         The epilogue warps also zero `out` before their first tile.
//   down kernel (split):  A = activation rows, B = 256 rows of w2[e] (K-major over H); epilogue:
//                         acc * routing weight -> bf16x2 vector reductions into out[token].
//                         Chained to the up kernel by programmatic dependent launch.
//   fused kernel (split == 0): per (row block, 128-wide H slice): up GEMM -> SwiGLU -> bf16
//                         activation tile kept in shared memory -> down GEMM against
//                         w2[e][:, slice] in 128-column chunks (double-buffered in TMEM) ->
//                         weighted fp32 vector reductions into a zeroed fp32 buffer [M, K] (split-K
//                         over H/128 slices, no bf16 rounding of partials); a small kernel chained
//                         by programmatic dependent launch then adds the buffer into `out`.
//
// All waits are bounded (ptx.cuh); no hardware barrier is used inside a role loop.
#include <stdio.h>

#include <algorithm>

#include "host_common.h"
#include "ptx.cuh"
#include "tile_sched.cuh"

namespace pmoe {

__device__ int g_status_bf16 = 0;

namespace {

constexpr int BM = 128;                          // rows per block (block_m)
constexpr int BK = 64;                           // bf16 elements in one 128-byte swizzled row
constexpr uint32_t A_BYTES = BM * BK * 2;        // 16 KB
constexpr uint32_t B_BYTES = 256 * BK * 2;       // 32 KB
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
constexpr uint32_t ACT_TILE_BYTES = 128 * 128 * 2;  // 128 rows x 128 bf16: two swizzled 16 KB halves
constexpr int MAX_STAGES = 4;
constexpr uint32_t TMEM_COLS = 512;
constexpr int GATHER_THREADS = 128;             // optional LSU gather warps at the end of the block
constexpr int MAX_THREADS = 64 + 8 * 32 + GATHER_THREADS;
constexpr uint32_t BAR_BYTES = 256;
constexpr uint32_t RED_ROW_BYTES = 256 + 16;     // down epilogue staging: 128 bf16 per row, padded against bank conflicts
constexpr uint32_t RED_STAGE_BYTES = 128 * RED_ROW_BYTES;

struct Args {
    const int32_t *sorted_ids;
    const int32_t *expert_ids;
    const int32_t *npp;
    const float *topk_weights;
    __nv_bfloat16 *out;
    float *acc32;    // fused kernel: fp32 accumulation buffer [M, K] the split-K partials are reduced into
    int M, K, N, H;
    int top_k;
    int sorted_num;
    int stages;
    int epi_warps;   // 4 or 8
    int zero_out;    // up kernel: clear `out` before the first tile
    int use_pdl;     // down kernel: wait for the primary grid before touching its results
    int bulk_reduce; // down kernels: epilogue reduces into `out` with cp.reduce.async.bulk from a staging tile
    int l2_ahead;    // producers prefetch weight tiles this many k-steps ahead of the ring into L2 (0 = off)
    int pregathered; // gate/up A operand: 0 = TMA gather4 from x, 1 = plain tiles from a row-gathered copy,
                     // 2 = gathered from x by four LSU warps (cp.async), no pre-pass
    const __nv_bfloat16 *x;   // mode 2: the activation matrix [M, K]
    // bpc == 2 with tail splitting: the pair kernels run the pairs of `pair_list` (both blocks hold routed rows),
    // the one-CTA kernels the first blocks of the pairs of `tail_list` (second block empty); counts = {pairs, tails}
    const int32_t *pair_list;
    const int32_t *tail_list;
    const int32_t *list_counts;
    const int32_t *live_rows;              // optional: rows of `out` in use (only those are zeroed)
    const unsigned long long *out_rows;    // optional: address of every row of `out` (down kernels, plain reductions)
    int down_ksplit; // one-CTA down kernel: split the k-range of its tiles when there are fewer tiles than CTAs
    int short_boxes; // one-CTA split kernels: row blocks with <= SHORT_ROWS routed rows move only those rows of
                     // the A operand and of the activation tile (the rest of a 128-row block is padding)
    __nv_bfloat16 *gu_out;   // optional [sorted_num, N]: the one-CTA gate/up kernels also store the gate | up
                             // pre-activations (bf16) for a later backward pass
};

constexpr int SHORT_ROWS = 32;
constexpr uint32_t SHORT_A_BYTES = SHORT_ROWS * 128;

// routed rows come first in a block, so the block is short when row SHORT_ROWS is already padding
__device__ __forceinline__ bool block_is_short(const Args &a, int blk, int what = 1) {
    return (a.short_boxes & what) && a.sorted_ids[blk * BM + SHORT_ROWS] < 0;
}

// rows of `out` the library has to zero
__device__ __forceinline__ int live_out_rows(const Args &a) {
    return a.live_rows ? max(0, min(a.M, *a.live_rows)) : a.M;
}
// destination of output row `tok`, columns from col0
__device__ __forceinline__ __nv_bfloat16 *out_row_ptr(const Args &a, int tok, int col0) {
    if (a.out_rows) return reinterpret_cast<__nv_bfloat16 *>(a.out_rows[tok]) + col0;
    return a.out + static_cast<size_t>(tok) * a.K + col0;
}

__device__ __forceinline__ int num_row_blocks(const Args &a) {
    int npp = *a.npp;
    npp = max(0, min(npp, a.sorted_num));
    return npp / BM;
}

// one-CTA kernels: number of row blocks to run and the block behind tile row i
__device__ __forceinline__ int num_tile_rows(const Args &a) {
    return a.tail_list ? a.list_counts[1] : num_row_blocks(a);
}
__device__ __forceinline__ int tile_row_block(const Args &a, int i) { return a.tail_list ? 2 * a.tail_list[i] : i; }

// bpc == 2: ordered lists of the pairs whose second block holds routed rows and of those whose second block is
// empty (the last pair of an expert with at most 128 rows left). One CTA; counts[0] = pairs, counts[1] = tails.
__global__ void __launch_bounds__(256)
classify_pairs_kernel(const int32_t *__restrict__ sorted_ids, const int32_t *__restrict__ npp, int sorted_num,
                      int32_t *__restrict__ pair_list, int32_t *__restrict__ tail_list, int32_t *__restrict__ counts) {
    __shared__ int s_warp[8];
    __shared__ int s_base[2];
    int n = *npp;
    n = max(0, min(n, sorted_num)) / (2 * BM);
    if (threadIdx.x == 0) s_base[0] = s_base[1] = 0;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i0 = 0; i0 < n; i0 += 256) {
        const int i = i0 + threadIdx.x;
        const bool in = i < n;
        const bool full = in && sorted_ids[(2 * i + 1) * BM] >= 0;
        const uint32_t b = __ballot_sync(0xffffffffu, full);
        if (lane == 0) s_warp[warp] = __popc(b);
        __syncthreads();
        int before = __popc(b & ((1u << lane) - 1u));
        for (int w = 0; w < warp; ++w) before += s_warp[w];
        int total = 0;
        for (int w = 0; w < 8; ++w) total += s_warp[w];
        const int base_full = s_base[0], base_tail = s_base[1];
        if (in) {
            if (full) pair_list[base_full + before] = i;
            else tail_list[base_tail + (threadIdx.x - before)] = i;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            s_base[0] = base_full + total;
            s_base[1] = base_tail + (min(256, n - i0) - total);
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        counts[0] = s_base[0];
        counts[1] = s_base[1];
    }
}

// Shared-memory carve-up (offsets from the 1024-byte aligned base):
//   [0, stages*48K) ring | [.., +32K) activation tile (up: store staging, fused: A operand) | barriers
struct Smem {
    uint32_t ring, act, bars;
    __device__ __forceinline__ uint32_t a(int s) const { return ring + s * STAGE_BYTES; }
    __device__ __forceinline__ uint32_t b(int s) const { return ring + s * STAGE_BYTES + A_BYTES; }
    __device__ __forceinline__ uint32_t full(int s) const { return bars + 8 * s; }
    __device__ __forceinline__ uint32_t empty(int s) const { return bars + 8 * (MAX_STAGES + s); }
    __device__ __forceinline__ uint32_t misc(int i) const { return bars + 8 * (2 * MAX_STAGES + i); }
    __device__ __forceinline__ uint32_t tmem_slot() const { return bars + 8 * (2 * MAX_STAGES + 12); }
};
__device__ __forceinline__ Smem carve(const uint8_t *raw, int stages, uint32_t extra) {
    Smem s;
    s.ring = (smem_u32(raw) + 1023u) & ~1023u;
    s.act = s.ring + stages * STAGE_BYTES;
    s.bars = s.act + extra;   // extra = activation tile (up / fused) or reduction staging (down) or 0
    return s;
}
size_t smem_bytes(int stages, uint32_t extra) {
    return 1024 + static_cast<size_t>(stages) * STAGE_BYTES + extra + BAR_BYTES;
}

// token rows for the four A-tile rows a producer lane gathers (rows 4*lane .. 4*lane+3 of the block)
__device__ __forceinline__ void gather_rows(const Args &a, int m_blk, int lane, int (&r)[4]) {
    const int4 p = *reinterpret_cast<const int4 *>(a.sorted_ids + m_blk * BM + 4 * lane);
    const int pr[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int tok = pr[i] >= 0 ? pr[i] / a.top_k : 0;  // padding rows read token 0, their result is dropped
        if (tok >= a.M) tok = 0;
        r[i] = tok;
    }
}

// After an abort: give the copies this producer issued a bounded time to land before the CTA exits.
__device__ __forceinline__ void drain_fills(const Smem &sm, int stages, long long issued) {
    const long long first = issued > stages ? issued - stages : 0;
    for (long long f = first; f < issued; ++f) {
        const uint32_t bar = sm.full(static_cast<int>(f % stages));
        const uint32_t parity = static_cast<uint32_t>((f / stages) & 1);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(bar, parity)) {
            if (globaltimer_ns() - t0 > 20000000ull) break;  // 20 ms
        }
    }
}

// SwiGLU epilogue for one 32-column chunk `c` (0..3) of a 128x128 activation tile: thread = row.
// Writes bf16 into the 128-byte-swizzled tile at `act` (two 16 KB halves of 64 columns).
template <bool kKeep = false>
__device__ __forceinline__ void swiglu_chunk_to_smem(uint32_t tmem_acc, uint32_t lane_base, int row, int c,
                                                     uint32_t act, __nv_bfloat16 *gu_row = nullptr, int H = 0) {
    float g[32], u[32];
    tmem_ld_32x32(g, tmem_addr(tmem_acc, lane_base, c * 32));
    tmem_ld_32x32(u, tmem_addr(tmem_acc, lane_base, 128 + c * 32));
    tmem_ld_wait();
    if (kKeep && gu_row) {   // keep the pre-activations: gate columns at gu_row, up columns H further (256-bit stores)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            uint32_t wg[8], wu[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                wg[q] = pack_bf16x2(g[16 * j + 2 * q], g[16 * j + 2 * q + 1]);
                wu[q] = pack_bf16x2(u[16 * j + 2 * q], u[16 * j + 2 * q + 1]);
            }
            st_global_v8(gu_row + c * 32 + 16 * j, wg);
            st_global_v8(gu_row + H + c * 32 + 16 * j, wu);
        }
    }
    const uint32_t row_addr = act + (c >> 1) * (ACT_TILE_BYTES / 2) + row * 128;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = j * 8 + e * 2;
            w[e] = pack_bf16x2(swiglu(g[i], u[i]), swiglu(g[i + 1], u[i + 1]));
        }
        const uint32_t chunk16 = static_cast<uint32_t>((c & 1) * 4 + j);
        st_shared_v4(row_addr + ((chunk16 ^ (row & 7)) << 4), w[0], w[1], w[2], w[3]);
    }
}

// acc chunk (32 columns) * weight -> bf16 -> four 16-byte vector reductions into out
__device__ __forceinline__ void reduce_chunk_to_out(uint32_t taddr, float wgt, __nv_bfloat16 *dst, bool valid) {
    float v[32];
    tmem_ld_32x32(v, taddr);
    tmem_ld_wait();
    if (valid) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            red_add_bf16x8(dst + j * 8, pack_bf16x2(wgt * v[j * 8 + 0], wgt * v[j * 8 + 1]),
                           pack_bf16x2(wgt * v[j * 8 + 2], wgt * v[j * 8 + 3]),
                           pack_bf16x2(wgt * v[j * 8 + 4], wgt * v[j * 8 + 5]),
                           pack_bf16x2(wgt * v[j * 8 + 6], wgt * v[j * 8 + 7]));
        }
    }
}

// acc chunk (32 columns) * weight -> eight 16-byte fp32 vector reductions into the fp32 accumulation buffer
__device__ __forceinline__ void reduce_chunk_to_acc32(uint32_t taddr, float wgt, float *dst, bool valid) {
    float v[32];
    tmem_ld_32x32(v, taddr);
    tmem_ld_wait();
    if (valid) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j * 4), "f"(wgt * v[j * 4 + 0]),
                         "f"(wgt * v[j * 4 + 1]), "f"(wgt * v[j * 4 + 2]), "f"(wgt * v[j * 4 + 3])
                         : "memory");
    }
}

// Down epilogue through the TMA engine: one accumulator row (thread = row) of 256 columns is scaled,
// rounded to bf16, staged 128 columns at a time in this thread's padded shared-memory row and added into
// out[token] by one 256-byte bulk reduction per half (instead of 16 scattered 16-byte reductions).
// Only the thread itself reads and writes its staging row, so its own bulk group is the only sync.
// `release` is called once the accumulator has been read completely.
template <typename Release>
__device__ __forceinline__ void bulk_reduce_row(uint32_t acc, uint32_t lane_base, uint32_t red_row, float wgt,
                                                __nv_bfloat16 *dst, bool valid, int cols, Release release) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        tma_store_wait_read<0>();   // this thread's previous reduction has finished reading the row
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float v[32];
            tmem_ld_32x32(v, tmem_addr(acc, lane_base, (half * 4 + q) * 32));
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j)
                st_shared_v4(red_row + q * 64 + j * 16, pack_bf16x2(wgt * v[j * 8 + 0], wgt * v[j * 8 + 1]),
                             pack_bf16x2(wgt * v[j * 8 + 2], wgt * v[j * 8 + 3]),
                             pack_bf16x2(wgt * v[j * 8 + 4], wgt * v[j * 8 + 5]),
                             pack_bf16x2(wgt * v[j * 8 + 6], wgt * v[j * 8 + 7]));
        }
        if (half == 1) release();
        fence_proxy_async_smem();
        if (valid && half * 128 < cols) bulk_reduce_add_bf16(dst + half * 128, red_row, 256);
        tma_store_commit();
    }
}

// out[i] += bf16(acc32[i]): last launch of the single-GEMM-launch pipeline (split == 0)
__global__ void __launch_bounds__(256)
finalize_acc32_kernel(const float *__restrict__ acc32, __nv_bfloat16 *__restrict__ out, long long n8, int use_pdl) {
    if (use_pdl) pdl_wait_primary();
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float4 a0 = __ldcg(reinterpret_cast<const float4 *>(acc32) + 2 * i);
        const float4 a1 = __ldcg(reinterpret_cast<const float4 *>(acc32) + 2 * i + 1);
        uint4 o = reinterpret_cast<const uint4 *>(out)[i];
        const __nv_bfloat162 *ob = reinterpret_cast<const __nv_bfloat162 *>(&o);
        uint4 r;
        r.x = pack_bf16x2(__low2float(ob[0]) + a0.x, __high2float(ob[0]) + a0.y);
        r.y = pack_bf16x2(__low2float(ob[1]) + a0.z, __high2float(ob[1]) + a0.w);
        r.z = pack_bf16x2(__low2float(ob[2]) + a1.x, __high2float(ob[2]) + a1.y);
        r.w = pack_bf16x2(__low2float(ob[3]) + a1.z, __high2float(ob[3]) + a1.w);
        reinterpret_cast<uint4 *>(out)[i] = r;
    }
}

// ---------------------------------------------------------------------------------------------
// optional pre-pass of the split pipeline: x_sorted[row] = x[token(row)] (one warp per row, 16-byte
// loads/stores) for the valid rows below num_tokens_post_padded; padding rows are left as they are.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ x_sorted, const Args a) {
    pdl_launch_dependents();   // the gate/up kernel may set itself up; it waits for this grid before loading
    const int warps_per_cta = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rows = num_row_blocks(a) * BM;
    const int chunks = a.K / 8;  // 16-byte chunks per row
    for (int row = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_cta) {
        const int pair = a.sorted_ids[row];
        const int tok = pair >= 0 ? pair / a.top_k : -1;
        // padding rows are not copied: whatever the workspace holds there only feeds accumulator rows that
        // no epilogue ever writes out (every output row depends on its own A row alone)
        if (tok < 0 || tok >= a.M) continue;
        const int4 *src = reinterpret_cast<const int4 *>(x + static_cast<size_t>(tok) * a.K);
        int4 *dst = reinterpret_cast<int4 *>(x_sorted + static_cast<size_t>(row) * a.K);
        for (int ch = lane; ch < chunks; ch += 32) dst[ch] = __ldg(src + ch);
    }
}

// ---------------------------------------------------------------------------------------------
// up kernel (split pipeline, first launch)
//   misc barriers: 0,1 tmem_full[2] | 2,3 tmem_empty[2] | 4 staged | 5 stage_free
// ---------------------------------------------------------------------------------------------
template <bool kKeep>
__global__ void __launch_bounds__(MAX_THREADS, 1)
moe_up_bf16_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w1,
                   const __grid_constant__ CUtensorMap map_act, const __grid_constant__ CUtensorMap map_x_short,
                   const __grid_constant__ CUtensorMap map_act_short, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const Smem sm = carve(smem_raw, a.stages, ACT_TILE_BYTES);
    int *status = &g_status_bf16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int epi_threads = a.epi_warps * 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(sm.full(s), a.pregathered == 2 ? 1 + GATHER_THREADS : 1);
            mbar_init(sm.empty(s), 1);
        }
        mbar_init(sm.misc(0), 1);
        mbar_init(sm.misc(1), 1);
        mbar_init(sm.misc(2), epi_threads);
        mbar_init(sm.misc(3), epi_threads);
        mbar_init(sm.misc(4), epi_threads);
        mbar_init(sm.misc(5), 1);
        fence_mbar_init();
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_w1);
        tma_prefetch_desc(&map_act);
    }
    if (warp == 1) tmem_alloc(sm.tmem_slot(), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(sm.tmem_slot()));

    // Dependents may be scheduled only now that this CTA holds its tensor memory: a dependent CTA that
    // shares this SM then blocks in its own allocation until this CTA has freed its columns, never the
    // other way round (it still waits for this whole grid before it reads any result).
    pdl_launch_dependents();

    if (a.use_pdl) pdl_wait_primary();   // launched as a programmatic dependent of the row-gather kernel

    const int m_blocks = num_tile_rows(a);
    const int n_tiles = a.H / 128;
    const int num_tiles = m_blocks * n_tiles;
    const int ksteps = a.K / BK;

    if (warp == 0) {
        // ---------------- producer: 32 lanes, lane l gathers rows 4l..4l+3 ----------------
        int s = 0;
        uint32_t ph = 0;
        long long issued = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const Coord c = tile_coord(t, m_blocks, n_tiles);
            const int mb = tile_row_block(a, c.m_blk);
            const int e = a.expert_ids[mb];
            int r[4];
            gather_rows(a, mb, lane, r);
            const int row_gate = e * a.N + c.n_tile * 128;
            const int row_up = row_gate + a.H;
            const bool short_a = a.pregathered != 2 && block_is_short(a, mb);
            const uint32_t fill_bytes =
                a.pregathered == 2 ? B_BYTES : (short_a ? B_BYTES + SHORT_A_BYTES : STAGE_BYTES);
            for (int ks = 0; ks < ksteps; ++ks) {
                if (lane == 0) ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane == 0) {
                    mbar_arrive_expect_tx(sm.full(s), fill_bytes);
                    tma_load_2d(sm.b(s), &map_w1, sm.full(s), ks * BK, row_gate);
                    tma_load_2d(sm.b(s) + B_BYTES / 2, &map_w1, sm.full(s), ks * BK, row_up);
                    if (a.pregathered == 1)
                        tma_load_2d(sm.a(s), short_a ? &map_x_short : &map_x, sm.full(s), ks * BK, mb * BM);
                    if (a.l2_ahead && ks + a.l2_ahead < ksteps) {
                        tma_prefetch_l2_2d(&map_w1, (ks + a.l2_ahead) * BK, row_gate);
                        tma_prefetch_l2_2d(&map_w1, (ks + a.l2_ahead) * BK, row_up);
                    }
                }
                __syncwarp();
                if (a.pregathered == 0 && (!short_a || lane < SHORT_ROWS / 4))   // short block: rows 0..31 only
                    tma_gather4(sm.a(s) + lane * 512, &map_x, sm.full(s), ks * BK, r[0], r[1], r[2], r[3]);
                ++issued;
                if (++s == a.stages) {
                    s = 0;
                    ph ^= 1;
                }
            }
        }
        if (!ok && lane == 0) drain_fills(sm, a.stages, issued);
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(128, 256);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
                const int buf = it & 1;
                ok = mbar_wait(sm.misc(2 + buf), ((it >> 1) & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * 256;
                for (int ks = 0; ks < ksteps; ++ks) {
                    ok = mbar_wait(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_f16(d, smem_desc_sw128(sm.a(s) + k * 32), smem_desc_sw128(sm.b(s) + k * 32), idesc,
                                 (ks | k) != 0);
                    umma_commit(sm.empty(s));
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit(sm.misc(buf));
            }
        }
        __syncwarp();
    } else if (warp >= 2 + a.epi_warps) {
        // ---------------- LSU gather warps (mode 2): A tile rows straight from x ----------------
        // 8 consecutive lanes copy the eight 16-byte chunks of one 128-byte row segment (a full line per
        // row, 4 rows per warp instruction); thread g serves rows (g>>3) + 16*i, i = 0..7.
        // cp.async writes shared memory through the generic proxy while tcgen05.mma reads it through the
        // async proxy, so each thread waits for its own copies of a slot (lagging `lag` slots behind the
        // ones it is issuing), fences the proxies, and only then arrives on the slot's full barrier.
        const int g = threadIdx.x - 64 - epi_threads;
        const int q = g >> 3, chunk = g & 7;
        const int lag = min(2, a.stages - 1);
        int s = 0, s_done = 0;
        uint32_t ph = 0;
        long long issued = 0, arrived = 0;
        auto publish = [&](int pending_allowed) {   // copies of all but the newest `pending_allowed` slots landed
            if (pending_allowed >= 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
            else if (pending_allowed == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
            else asm volatile("cp.async.wait_group 0;" ::: "memory");
            fence_proxy_async_smem();
            while (arrived < issued - pending_allowed) {
                mbar_arrive(sm.full(s_done));
                if (++s_done == a.stages) s_done = 0;
                ++arrived;
            }
        };
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const Coord c = tile_coord(t, m_blocks, n_tiles);
            const int mb = tile_row_block(a, c.m_blk);
            const char *src[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int pair = a.sorted_ids[mb * BM + q + 16 * i];
                int tok = pair >= 0 ? pair / a.top_k : 0;
                if (tok >= a.M) tok = 0;
                src[i] = reinterpret_cast<const char *>(a.x + static_cast<size_t>(tok) * a.K) + chunk * 16;
            }
            for (int ks = 0; ks < ksteps; ++ks) {
                ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                if (!ok) break;
                // (q + 16 i) & 7 == q & 7: every row of this thread uses the same swizzled chunk slot
                const uint32_t dst = sm.a(s) + q * 128 + ((chunk ^ (q & 7)) << 4);
#pragma unroll
                for (int i = 0; i < 8; ++i) cp_async_16(dst + i * 16 * 128, src[i] + ks * 128);
                asm volatile("cp.async.commit_group;" ::: "memory");
                ++issued;
                if (++s == a.stages) {
                    s = 0;
                    ph ^= 1;
                }
                if (issued - arrived > lag) publish(lag);
            }
        }
        publish(0);
        cp_async_wait_all();
    } else {
        // ---------------- epilogue: thread = accumulator row ----------------
        const int ew = warp - 2;
        const int et = threadIdx.x - 64;
        const uint32_t lane_base = (warp & 3) * 32;  // TMEM lane quarter this warp may read
        const int row = lane_base + lane;
        const int ncg = a.epi_warps / 4;             // column groups (1 or 2)
        const int cg = ew / 4;
        if (a.zero_out) {
            int4 *o4 = reinterpret_cast<int4 *>(a.out);
            const long long n4 = static_cast<long long>(live_out_rows(a)) * a.K / 8;
            const int4 z = make_int4(0, 0, 0, 0);
            for (long long i = static_cast<long long>(blockIdx.x) * epi_threads + et; i < n4;
                 i += static_cast<long long>(gridDim.x) * epi_threads)
                o4[i] = z;
        }
        int it = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            const Coord c = tile_coord(t, m_blocks, n_tiles);
            const int mb = tile_row_block(a, c.m_blk);
            const int buf = it & 1;
            if (!mbar_wait(sm.misc(buf), (it >> 1) & 1, status, ST_TIMEOUT_TMEM_FULL)) break;
            if (!mbar_wait(sm.misc(5), (it & 1) ^ 1, status, ST_TIMEOUT_ACT)) break;  // staging tile free
            tc_fence_after();
            const uint32_t acc = tmem_base + buf * 256;
            __nv_bfloat16 *gu_row =
                kKeep ? a.gu_out + (static_cast<size_t>(mb) * BM + row) * a.N + c.n_tile * 128 : nullptr;
            for (int ch = cg * (4 / ncg); ch < (cg + 1) * (4 / ncg); ++ch)
                swiglu_chunk_to_smem<kKeep>(acc, lane_base, row, ch, sm.act, gu_row, a.H);
            tc_fence_before();
            mbar_arrive(sm.misc(2 + buf));  // accumulator drained
            fence_proxy_async_smem();
            mbar_arrive(sm.misc(4));        // staging tile written
            if (et == 0) {
                if (!mbar_wait(sm.misc(4), it & 1, status, ST_TIMEOUT_ACT)) break;
                const CUtensorMap *st = block_is_short(a, mb, 2) ? &map_act_short : &map_act;
                tma_store_2d(st, sm.act, c.n_tile * 128, mb * BM);
                tma_store_2d(st, sm.act + ACT_TILE_BYTES / 2, c.n_tile * 128 + 64, mb * BM);
                tma_store_commit();
                tma_store_wait_read<0>();
                mbar_arrive(sm.misc(5));
            }
        }
        if (et == 0) tma_store_wait<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// gate/up kernel with TWO row blocks per tile (one CTA, no counterpart in the reference): the consecutive
// blocks 2q and 2q+1, when they belong to one expert, share every weight slot of the ring - 64 KB per
// k-step feed 2 x (128 x 256 x 64) MACs instead of 2 x 48 KB, the same operand traffic per MAC as the CTA
// pairs but on routing tables padded to 128 rows and with the in-kernel LSU row gather. Block 2q
// accumulates in TMEM columns [0,256), block 2q+1 in [256,512); the epilogue drains them one after the
// other and the next tile's MMAs start on each accumulator as soon as it is free. Blocks 2q, 2q+1 of
// different experts (and an odd last block) run as single-block passes with their own weight loads.
//   misc barriers: 0,1 tmem_full[acc] | 2,3 tmem_empty[acc] | 4 staged | 5 stage_free
// ---------------------------------------------------------------------------------------------
constexpr uint32_t DUAL_STAGE_BYTES = 2 * A_BYTES + B_BYTES;   // 64 KB
constexpr int DUAL_MAX_STAGES = 3;

struct SmemDual {
    uint32_t ring, act, bars;
    __device__ __forceinline__ uint32_t a(int s, int h) const { return ring + s * DUAL_STAGE_BYTES + h * A_BYTES; }
    __device__ __forceinline__ uint32_t b(int s) const { return ring + s * DUAL_STAGE_BYTES + 2 * A_BYTES; }
    __device__ __forceinline__ uint32_t full(int s) const { return bars + 8 * s; }
    __device__ __forceinline__ uint32_t empty(int s) const { return bars + 8 * (DUAL_MAX_STAGES + s); }
    __device__ __forceinline__ uint32_t misc(int i) const { return bars + 8 * (2 * DUAL_MAX_STAGES + i); }
    __device__ __forceinline__ uint32_t tmem_slot() const { return bars + 8 * (2 * DUAL_MAX_STAGES + 8); }
};
__device__ __forceinline__ SmemDual carve_dual(const uint8_t *raw, int stages) {
    SmemDual s;
    s.ring = (smem_u32(raw) + 1023u) & ~1023u;
    s.act = s.ring + stages * DUAL_STAGE_BYTES;
    s.bars = s.act + ACT_TILE_BYTES;
    return s;
}
size_t smem_bytes_dual(int stages) { return 1024 + static_cast<size_t>(stages) * DUAL_STAGE_BYTES + ACT_TILE_BYTES + BAR_BYTES; }

struct Pass {
    int blk[2];   // row blocks of the pass (blk[1] = -1 for a single-block pass)
    int nblk;
    int expert;
};
// the one or two passes of tile pair q; identical in every role of the CTA
__device__ __forceinline__ int tile_passes(const Args &a, int q, int m_blocks, Pass (&p)[2]) {
    const int b0 = 2 * q, b1 = b0 + 1;
    const int e0 = a.expert_ids[b0];
    p[0].blk[0] = b0;
    p[0].blk[1] = -1;
    p[0].nblk = 1;
    p[0].expert = e0;
    if (b1 >= m_blocks) return 1;
    const int e1 = a.expert_ids[b1];
    if (e1 == e0) {
        p[0].blk[1] = b1;
        p[0].nblk = 2;
        return 1;
    }
    p[1].blk[0] = b1;
    p[1].blk[1] = -1;
    p[1].nblk = 1;
    p[1].expert = e1;
    return 2;
}

template <bool kKeep>
__global__ void __launch_bounds__(MAX_THREADS, 1)
moe_up_dual_bf16_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w1,
                        const __grid_constant__ CUtensorMap map_act, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const SmemDual sm = carve_dual(smem_raw, a.stages);
    int *status = &g_status_bf16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int epi_threads = a.epi_warps * 32;
    const bool lsu = a.pregathered == 2;
    const int gather_threads = static_cast<int>(blockDim.x) - 64 - epi_threads;   // 0, 128 or 256

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(sm.full(s), lsu ? 1 + gather_threads : 1);
            mbar_init(sm.empty(s), 1);
        }
        mbar_init(sm.misc(0), 1);
        mbar_init(sm.misc(1), 1);
        mbar_init(sm.misc(2), epi_threads);
        mbar_init(sm.misc(3), epi_threads);
        mbar_init(sm.misc(4), epi_threads);
        mbar_init(sm.misc(5), 1);
        fence_mbar_init();
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_w1);
        tma_prefetch_desc(&map_act);
    }
    if (warp == 1) tmem_alloc(sm.tmem_slot(), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(sm.tmem_slot()));

    // Dependents may be scheduled only now that this CTA holds its tensor memory: a dependent CTA that
    // shares this SM then blocks in its own allocation until this CTA has freed its columns, never the
    // other way round (it still waits for this whole grid before it reads any result).
    pdl_launch_dependents();

    if (a.use_pdl) pdl_wait_primary();   // launched as a programmatic dependent of the row-gather kernel

    const int m_blocks = num_row_blocks(a);
    const int m_pairs = (m_blocks + 1) / 2;
    const int n_tiles = a.H / 128;
    const int num_tiles = m_pairs * n_tiles;
    const int ksteps = a.K / BK;

    if (warp == 0) {
        // ---------------- producer: weight slots (and the pre-gathered A tiles) by TMA ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const Coord c = tile_coord(t, m_pairs, n_tiles);
                Pass ps[2];
                const int np = tile_passes(a, c.m_blk, m_blocks, ps);
                for (int pi = 0; pi < np && ok; ++pi) {
                    const Pass &p = ps[pi];
                    const int row_gate = p.expert * a.N + c.n_tile * 128;
                    const int row_up = row_gate + a.H;
                    const uint32_t bytes = B_BYTES + (lsu ? 0u : static_cast<uint32_t>(p.nblk) * A_BYTES);
                    for (int ks = 0; ks < ksteps; ++ks) {
                        ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                        if (!ok) break;
                        mbar_arrive_expect_tx(sm.full(s), bytes);
                        tma_load_2d(sm.b(s), &map_w1, sm.full(s), ks * BK, row_gate);
                        tma_load_2d(sm.b(s) + B_BYTES / 2, &map_w1, sm.full(s), ks * BK, row_up);
                        if (!lsu) {
                            tma_load_2d(sm.a(s, 0), &map_x, sm.full(s), ks * BK, p.blk[0] * BM);
                            if (p.nblk == 2) tma_load_2d(sm.a(s, 1), &map_x, sm.full(s), ks * BK, p.blk[1] * BM);
                        }
                        if (++s == a.stages) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(128, 256);
            int s = 0;
            uint32_t ph = 0;
            uint32_t uses[2] = {0, 0};   // completed passes per accumulator
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const Coord c = tile_coord(t, m_pairs, n_tiles);
                Pass ps[2];
                const int np = tile_passes(a, c.m_blk, m_blocks, ps);
                for (int pi = 0; pi < np && ok; ++pi) {
                    const int nblk = ps[pi].nblk;
                    ok = mbar_wait(sm.misc(2), (uses[0] & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                    if (!ok) break;
                    tc_fence_after();
                    for (int ks = 0; ks < ksteps; ++ks) {
                        ok = mbar_wait(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_f16(tmem_base, smem_desc_sw128(sm.a(s, 0) + k * 32), smem_desc_sw128(sm.b(s) + k * 32),
                                     idesc, (ks | k) != 0);
                        if (nblk == 2) {
                            if (ks == 0) {   // the second accumulator is waited for as late as possible
                                ok = mbar_wait(sm.misc(3), (uses[1] & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                                if (!ok) break;
                                tc_fence_after();
                            }
#pragma unroll
                            for (int k = 0; k < BK / 16; ++k)
                                umma_f16(tmem_base + 256, smem_desc_sw128(sm.a(s, 1) + k * 32),
                                         smem_desc_sw128(sm.b(s) + k * 32), idesc, (ks | k) != 0);
                        }
                        umma_commit(sm.empty(s));
                        if (++s == a.stages) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                    if (!ok) break;
                    umma_commit(sm.misc(0));
                    ++uses[0];
                    if (nblk == 2) {
                        umma_commit(sm.misc(1));
                        ++uses[1];
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp >= 2 + a.epi_warps) {
        // ---------------- LSU gather warps (mode 2): the A rows of both blocks straight from x ----------------
        // as in moe_up_bf16_kernel: 8 lanes per 128-byte row segment, a thread serves rows (g>>3) + 16*i of a
        // block, lagged wait_group + proxy fence before its arrival on the slot's full barrier. With eight
        // gather warps the first four serve block 2q and the last four block 2q+1; with four, every thread
        // serves both blocks.
        const int g = (threadIdx.x - 64 - epi_threads) & 127;
        const int serve = gather_threads == 256 ? (static_cast<int>(threadIdx.x) - 64 - epi_threads) >> 7 : -1;   // -1: both blocks
        const int q = g >> 3, chunk = g & 7;
        // a slot is published while the NEXT one is being issued: with three slots a lag of two would make
        // every k-step wait for the MMAs of the previous one
        const int lag = min(1, a.stages - 1);
        int s = 0, s_done = 0;
        uint32_t ph = 0;
        long long issued = 0, arrived = 0;
        auto publish = [&](int pending_allowed) {
            if (pending_allowed >= 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
            else if (pending_allowed == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
            else asm volatile("cp.async.wait_group 0;" ::: "memory");
            fence_proxy_async_smem();
            while (arrived < issued - pending_allowed) {
                mbar_arrive(sm.full(s_done));
                if (++s_done == a.stages) s_done = 0;
                ++arrived;
            }
        };
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const Coord c = tile_coord(t, m_pairs, n_tiles);
            Pass ps[2];
            const int np = tile_passes(a, c.m_blk, m_blocks, ps);
            for (int pi = 0; pi < np && ok; ++pi) {
                const Pass &p = ps[pi];
                const char *src[2][8];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int pair = h < p.nblk ? a.sorted_ids[p.blk[h] * BM + q + 16 * i] : -1;
                        int tok = pair >= 0 ? pair / a.top_k : 0;
                        if (tok >= a.M) tok = 0;
                        src[h][i] = reinterpret_cast<const char *>(a.x + static_cast<size_t>(tok) * a.K) + chunk * 16;
                    }
                }
                for (int ks = 0; ks < ksteps; ++ks) {
                    ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                    if (!ok) break;
                    const uint32_t off = q * 128 + ((chunk ^ (q & 7)) << 4);
                    if (serve != 1) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) cp_async_16(sm.a(s, 0) + off + i * 16 * 128, src[0][i] + ks * 128);
                    }
                    if (p.nblk == 2 && serve != 0) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) cp_async_16(sm.a(s, 1) + off + i * 16 * 128, src[1][i] + ks * 128);
                    }
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    ++issued;
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                    if (issued - arrived > lag) publish(lag);
                }
            }
        }
        publish(0);
        cp_async_wait_all();
    } else {
        // ---------------- epilogue: thread = accumulator row, one accumulator after the other ----------------
        const int ew = warp - 2;
        const int et = threadIdx.x - 64;
        const uint32_t lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;
        const int ncg = a.epi_warps / 4;
        const int cg = ew / 4;
        if (a.zero_out) {
            int4 *o4 = reinterpret_cast<int4 *>(a.out);
            const long long n4 = static_cast<long long>(live_out_rows(a)) * a.K / 8;
            const int4 z = make_int4(0, 0, 0, 0);
            for (long long i = static_cast<long long>(blockIdx.x) * epi_threads + et; i < n4;
                 i += static_cast<long long>(gridDim.x) * epi_threads)
                o4[i] = z;
        }
        uint32_t uses[2] = {0, 0};
        uint32_t stores = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const Coord c = tile_coord(t, m_pairs, n_tiles);
            Pass ps[2];
            const int np = tile_passes(a, c.m_blk, m_blocks, ps);
            for (int pi = 0; pi < np && ok; ++pi) {
                for (int h = 0; h < ps[pi].nblk && ok; ++h) {
                    ok = mbar_wait(sm.misc(h), uses[h] & 1, status, ST_TIMEOUT_TMEM_FULL) &&
                         mbar_wait(sm.misc(5), (stores & 1) ^ 1, status, ST_TIMEOUT_ACT);   // staging tile free
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t acc = tmem_base + h * 256;
                    __nv_bfloat16 *gu_row =
                        kKeep ? a.gu_out + (static_cast<size_t>(ps[pi].blk[h]) * BM + row) * a.N + c.n_tile * 128
                              : nullptr;
                    for (int ch = cg * (4 / ncg); ch < (cg + 1) * (4 / ncg); ++ch)
                        swiglu_chunk_to_smem<kKeep>(acc, lane_base, row, ch, sm.act, gu_row, a.H);
                    tc_fence_before();
                    mbar_arrive(sm.misc(2 + h));   // accumulator drained
                    fence_proxy_async_smem();
                    mbar_arrive(sm.misc(4));       // staging tile written
                    if (et == 0) {
                        ok = mbar_wait(sm.misc(4), stores & 1, status, ST_TIMEOUT_ACT);
                        if (!ok) break;
                        tma_store_2d(&map_act, sm.act, c.n_tile * 128, ps[pi].blk[h] * BM);
                        tma_store_2d(&map_act, sm.act + ACT_TILE_BYTES / 2, c.n_tile * 128 + 64, ps[pi].blk[h] * BM);
                        tma_store_commit();
                        tma_store_wait_read<0>();
                        mbar_arrive(sm.misc(5));
                    }
                    ++uses[h];
                    ++stores;
                }
            }
        }
        if (et == 0) tma_store_wait<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// down kernel (split pipeline, second launch)
//   misc barriers: 0,1 tmem_full[2] | 2,3 tmem_empty[2]
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(MAX_THREADS, 1)
moe_down_bf16_kernel(const __grid_constant__ CUtensorMap map_act, const __grid_constant__ CUtensorMap map_w2,
                     const __grid_constant__ CUtensorMap map_act_short, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const Smem sm = carve(smem_raw, a.stages, a.bulk_reduce ? RED_STAGE_BYTES : 0u);
    int *status = &g_status_bf16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int epi_threads = a.epi_warps * 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        mbar_init(sm.misc(0), 1);
        mbar_init(sm.misc(1), 1);
        mbar_init(sm.misc(2), a.bulk_reduce ? 128 : epi_threads);   // the bulk epilogue runs on 4 warps
        mbar_init(sm.misc(3), a.bulk_reduce ? 128 : epi_threads);
        fence_mbar_init();
        tma_prefetch_desc(&map_act);
        tma_prefetch_desc(&map_w2);
    }
    if (warp == 1) tmem_alloc(sm.tmem_slot(), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(sm.tmem_slot()));

    if (a.use_pdl) pdl_wait_primary();  // activations and the zeroed `out` come from the up kernel

    const int m_blocks = num_tile_rows(a);
    const int n_tiles = (a.K + 255) / 256;
    const int ksteps_all = a.H / BK;
    // Few tiles for many SMs (the single-block tails of the bpc = 2 pipeline: a handful of row blocks x K/256
    // column tiles): cut every tile's k-range into `ksplit` parts run as tiles of their own. The epilogue ADDS into
    // `out` anyway, so the partial products need no extra reduction.
    int ksplit = 1;
    if (a.down_ksplit && m_blocks * n_tiles > 0) ksplit = max(1, min(min(4, ksteps_all), static_cast<int>(gridDim.x) / (m_blocks * n_tiles)));
    const int kchunk = (ksteps_all + ksplit - 1) / ksplit;
    ksplit = (ksteps_all + kchunk - 1) / kchunk;   // no empty part: an accumulator without MMAs must never be added
    const int base_tiles = m_blocks * n_tiles;
    const int num_tiles = base_tiles * ksplit;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            long long issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const Coord c = tile_coord(t % base_tiles, m_blocks, n_tiles);
                const int ks0 = (t / base_tiles) * kchunk, ks1 = min(ksteps_all, ks0 + kchunk);
                const int mb = tile_row_block(a, c.m_blk);
                const int e = a.expert_ids[mb];
                const int w2_row = e * a.K + c.n_tile * 256;
                const bool short_a = block_is_short(a, mb);
                for (int ks = ks0; ks < ks1; ++ks) {
                    ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_arrive_expect_tx(sm.full(s), short_a ? B_BYTES + SHORT_A_BYTES : STAGE_BYTES);
                    tma_load_2d(sm.a(s), short_a ? &map_act_short : &map_act, sm.full(s), ks * BK, mb * BM);
                    tma_load_2d(sm.b(s), &map_w2, sm.full(s), ks * BK, w2_row);
                    if (a.l2_ahead && ks + a.l2_ahead < ks1) tma_prefetch_l2_2d(&map_w2, (ks + a.l2_ahead) * BK, w2_row);
                    ++issued;
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
            if (!ok) drain_fills(sm, a.stages, issued);
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(128, 256);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
                const int buf = it & 1;
                ok = mbar_wait(sm.misc(2 + buf), ((it >> 1) & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * 256;
                const int ks0 = (t / base_tiles) * kchunk, ks1 = min(ksteps_all, ks0 + kchunk);
                for (int ks = ks0; ks < ks1; ++ks) {
                    ok = mbar_wait(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_f16(d, smem_desc_sw128(sm.a(s) + k * 32), smem_desc_sw128(sm.b(s) + k * 32), idesc,
                                 (ks != ks0) || (k != 0));
                    umma_commit(sm.empty(s));
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit(sm.misc(buf));
            }
        }
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const uint32_t lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;
        const int ncg = a.epi_warps / 4;
        const int cg = ew / 4;
        int it = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            const Coord c = tile_coord(t % base_tiles, m_blocks, n_tiles);
            const int mb = tile_row_block(a, c.m_blk);
            const int buf = it & 1;
            const int pair = a.sorted_ids[mb * BM + row];
            const int tok = pair >= 0 ? pair / a.top_k : 0;
            const bool valid = pair >= 0 && tok < a.M;
            const float wgt = valid ? a.topk_weights[pair] : 0.f;
            const int col0 = c.n_tile * 256;
            __nv_bfloat16 *dst = valid ? out_row_ptr(a, tok, col0) : a.out;
            const int cols = min(256, a.K - col0);
            if (a.bulk_reduce && ew >= 4) break;   // warps beyond the first four idle in the bulk epilogue
            if (!mbar_wait(sm.misc(buf), (it >> 1) & 1, status, ST_TIMEOUT_TMEM_FULL)) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + buf * 256;
            if (a.bulk_reduce) {
                bulk_reduce_row(acc, lane_base, sm.act + row * RED_ROW_BYTES, wgt, dst, valid, cols, [&] {
                    tc_fence_before();
                    mbar_arrive(sm.misc(2 + buf));
                });
                continue;
            }
            for (int ch = cg * (8 / ncg); ch < (cg + 1) * (8 / ncg); ++ch)
                reduce_chunk_to_out(tmem_addr(acc, lane_base, ch * 32), wgt, dst + ch * 32,
                                    valid && ch * 32 < cols);
            tc_fence_before();
            mbar_arrive(sm.misc(2 + buf));
        }
        if (a.bulk_reduce) tma_store_wait<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// fused kernel (split == 0): one launch, activation tile stays on chip, split-K over H/128 slices
//   TMEM: [0,256) gate|up accumulator, [256,384) and [384,512) down accumulators (128 columns each)
//   misc barriers: 0 up_full | 1 up_empty | 2 act_ready | 3 act_free | 4,5 dn_full[2] | 6,7 dn_empty[2]
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(MAX_THREADS, 1)
moe_fused_bf16_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w1,
                      const __grid_constant__ CUtensorMap map_w2, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const Smem sm = carve(smem_raw, a.stages, ACT_TILE_BYTES);
    int *status = &g_status_bf16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int epi_threads = a.epi_warps * 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        mbar_init(sm.misc(0), 1);
        mbar_init(sm.misc(1), epi_threads);
        mbar_init(sm.misc(2), epi_threads);
        mbar_init(sm.misc(3), 1);
        mbar_init(sm.misc(4), 1);
        mbar_init(sm.misc(5), 1);
        mbar_init(sm.misc(6), epi_threads);
        mbar_init(sm.misc(7), epi_threads);
        fence_mbar_init();
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_w1);
        tma_prefetch_desc(&map_w2);
    }
    if (warp == 1) tmem_alloc(sm.tmem_slot(), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(sm.tmem_slot()));

    // Dependents may be scheduled only now that this CTA holds its tensor memory: a dependent CTA that
    // shares this SM then blocks in its own allocation until this CTA has freed its columns, never the
    // other way round (it still waits for this whole grid before it reads any result).
    pdl_launch_dependents();

    const int m_blocks = num_row_blocks(a);
    const int n_tiles = a.H / 128;          // H slices
    const int num_tiles = m_blocks * n_tiles;
    const int ksteps = a.K / BK;
    const int dn_chunks = a.K / 128;        // 128 output columns per down chunk

    if (warp == 0) {
        int s = 0;
        uint32_t ph = 0;
        long long issued = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const Coord c = tile_coord(t, m_blocks, n_tiles);
            const int e = a.expert_ids[c.m_blk];
            int r[4];
            gather_rows(a, c.m_blk, lane, r);
            const int row_gate = e * a.N + c.n_tile * 128;
            const int row_up = row_gate + a.H;
            for (int ks = 0; ks < ksteps; ++ks) {
                if (lane == 0) ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane == 0) {
                    mbar_arrive_expect_tx(sm.full(s), STAGE_BYTES);
                    tma_load_2d(sm.b(s), &map_w1, sm.full(s), ks * BK, row_gate);
                    tma_load_2d(sm.b(s) + B_BYTES / 2, &map_w1, sm.full(s), ks * BK, row_up);
                    if (a.pregathered) tma_load_2d(sm.a(s), &map_x, sm.full(s), ks * BK, c.m_blk * BM);
                    if (a.l2_ahead && ks + a.l2_ahead < ksteps) {
                        tma_prefetch_l2_2d(&map_w1, (ks + a.l2_ahead) * BK, row_gate);
                        tma_prefetch_l2_2d(&map_w1, (ks + a.l2_ahead) * BK, row_up);
                    }
                }
                __syncwarp();
                if (!a.pregathered)
                    tma_gather4(sm.a(s) + lane * 512, &map_x, sm.full(s), ks * BK, r[0], r[1], r[2], r[3]);
                ++issued;
                if (++s == a.stages) {
                    s = 0;
                    ph ^= 1;
                }
            }
            if (!ok) break;
            // down phase: w2[e][chunk*128 .. +128, slice*128 + kh*64 .. +64] -> B part of a slot
            for (int ch = 0; ch < dn_chunks && ok; ++ch) {
                for (int kh = 0; kh < 2; ++kh) {
                    if (lane == 0) ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    if (lane == 0) {
                        mbar_arrive_expect_tx(sm.full(s), B_BYTES / 2);
                        tma_load_2d(sm.b(s), &map_w2, sm.full(s), c.n_tile * 128 + kh * 64, e * a.K + ch * 128);
                    }
                    ++issued;
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
        if (!ok && lane == 0) drain_fills(sm, a.stages, issued);
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_up = idesc_bf16_f32(128, 256);
            constexpr uint32_t idesc_dn = idesc_bf16_f32(128, 128);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            long long dn_it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
                ok = mbar_wait(sm.misc(1), (it & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                for (int ks = 0; ks < ksteps; ++ks) {
                    ok = mbar_wait(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_f16(tmem_base, smem_desc_sw128(sm.a(s) + k * 32), smem_desc_sw128(sm.b(s) + k * 32),
                                 idesc_up, (ks | k) != 0);
                    umma_commit(sm.empty(s));
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(sm.misc(0));
                ok = mbar_wait(sm.misc(2), it & 1, status, ST_TIMEOUT_ACT);  // activation tile in smem
                if (!ok) break;
                tc_fence_after();
                for (int ch = 0; ch < dn_chunks && ok; ++ch, ++dn_it) {
                    const int b = static_cast<int>(dn_it & 1);
                    ok = mbar_wait(sm.misc(6 + b), static_cast<uint32_t>(((dn_it >> 1) & 1) ^ 1), status,
                                   ST_TIMEOUT_TMEM_EMPTY);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d = tmem_base + 256 + b * 128;
                    for (int kh = 0; kh < 2; ++kh) {
                        ok = mbar_wait(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_f16(d, smem_desc_sw128(sm.act + kh * (ACT_TILE_BYTES / 2) + k * 32),
                                     smem_desc_sw128(sm.b(s) + k * 32), idesc_dn, (kh | k) != 0);
                        umma_commit(sm.empty(s));
                        if (++s == a.stages) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                    if (ok) umma_commit(sm.misc(4 + b));
                }
                if (ok) umma_commit(sm.misc(3));  // every MMA that reads the activation tile is done
            }
        }
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const uint32_t lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;
        const int ncg = a.epi_warps / 4;
        const int cg = ew / 4;
        int it = 0;
        long long dn_it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
            const Coord c = tile_coord(t, m_blocks, n_tiles);
            const int pair = a.sorted_ids[c.m_blk * BM + row];
            const int tok = pair >= 0 ? pair / a.top_k : 0;
            const bool valid = pair >= 0 && tok < a.M;
            const float wgt = valid ? a.topk_weights[pair] : 0.f;
            float *dst = a.acc32 + static_cast<size_t>(valid ? tok : 0) * a.K;
            if (!mbar_wait(sm.misc(0), it & 1, status, ST_TIMEOUT_TMEM_FULL)) break;
            if (!mbar_wait(sm.misc(3), (it & 1) ^ 1, status, ST_TIMEOUT_ACT)) break;  // act tile reusable
            tc_fence_after();
            for (int ch = cg * (4 / ncg); ch < (cg + 1) * (4 / ncg); ++ch)
                swiglu_chunk_to_smem(tmem_base, lane_base, row, ch, sm.act);
            tc_fence_before();
            mbar_arrive(sm.misc(1));
            fence_proxy_async_smem();
            mbar_arrive(sm.misc(2));
            for (int ch = 0; ch < dn_chunks; ++ch, ++dn_it) {
                const int b = static_cast<int>(dn_it & 1);
                ok = mbar_wait(sm.misc(4 + b), static_cast<uint32_t>((dn_it >> 1) & 1), status,
                               ST_TIMEOUT_TMEM_FULL);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + 256 + b * 128;
                for (int q = cg * (4 / ncg); q < (cg + 1) * (4 / ncg); ++q)
                    reduce_chunk_to_acc32(tmem_addr(acc, lane_base, q * 32), wgt, dst + ch * 128 + q * 32, valid);
                tc_fence_before();
                mbar_arrive(sm.misc(6 + b));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// bpc == 2: CTA pairs (cluster of 2) with tcgen05 cta_group::2 MMAs, M = 256 per pair
//
// A pair owns two consecutive 128-row blocks (same expert: moe_align pads experts to 256 rows when
// bpc == 2) x one 256-column tile. Each CTA loads ITS 128 rows of A and ITS half of the B tile (up
// kernel: CTA 0 the gate rows, CTA 1 the up rows; down kernel: 128 of the 256 w2 rows each), so a CTA
// pulls 32 KB per k-step for 128x256x64 MACs instead of 48 KB - two thirds of the L2->SM traffic.
// Plain TMA tile loads only (no multicast). The even CTA issues the MMAs for both; its `full`
// barriers collect the bytes of both CTAs' loads; ring slots and accumulators are released to both
// CTAs by multicast tcgen05.commit; both CTAs' epilogue warps arrive on the even CTA's tmem_empty.
//   misc barriers: 0,1 tmem_full[2] | 2,3 tmem_empty[2] (leader) | 4 staged | 5 stage_free (up only)
// ---------------------------------------------------------------------------------------------
constexpr uint32_t PAIR_STAGE_BYTES = A_BYTES + B_BYTES / 2;   // 32 KB per CTA and slot
constexpr int PAIR_MAX_STAGES = 6;
constexpr int ST_BAD_PAIR = 8;                                 // the two blocks of a pair differ in expert

struct SmemPair {
    uint32_t ring, act, bars;
    __device__ __forceinline__ uint32_t a(int s) const { return ring + s * PAIR_STAGE_BYTES; }
    __device__ __forceinline__ uint32_t b(int s) const { return ring + s * PAIR_STAGE_BYTES + A_BYTES; }
    __device__ __forceinline__ uint32_t full(int s) const { return bars + 8 * s; }
    __device__ __forceinline__ uint32_t empty(int s) const { return bars + 8 * (PAIR_MAX_STAGES + s); }
    __device__ __forceinline__ uint32_t misc(int i) const { return bars + 8 * (2 * PAIR_MAX_STAGES + i); }
    __device__ __forceinline__ uint32_t tmem_slot() const { return bars + 8 * (2 * PAIR_MAX_STAGES + 12); }
};
__device__ __forceinline__ SmemPair carve_pair(const uint8_t *raw, int stages, uint32_t extra) {
    SmemPair s;
    s.ring = (smem_u32(raw) + 1023u) & ~1023u;
    s.act = s.ring + stages * PAIR_STAGE_BYTES;
    s.bars = s.act + extra;
    return s;
}
size_t smem_bytes_pair(int stages, uint32_t extra) {
    return 1024 + static_cast<size_t>(stages) * PAIR_STAGE_BYTES + extra + BAR_BYTES;
}

template <bool kUp, bool kKeep = false>
__global__ void __launch_bounds__(MAX_THREADS, 1)
moe_pair_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_act, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const SmemPair sm = carve_pair(smem_raw, a.stages, kUp ? ACT_TILE_BYTES : (a.bulk_reduce ? RED_STAGE_BYTES : 0u));
    int *status = &g_status_bf16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int epi_threads = a.epi_warps * 32;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        mbar_init(sm.misc(0), 1);
        mbar_init(sm.misc(1), 1);
        mbar_init(sm.misc(2), 2 * ((!kUp && a.bulk_reduce) ? 128 : epi_threads));
        mbar_init(sm.misc(3), 2 * ((!kUp && a.bulk_reduce) ? 128 : epi_threads));
        mbar_init(sm.misc(4), epi_threads);
        mbar_init(sm.misc(5), 1);
        fence_mbar_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
        if (kUp) tma_prefetch_desc(&map_act);
    }
    if (warp == 1) tmem_alloc_pair(sm.tmem_slot(), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();      // both CTAs' barriers are initialised and both halves of TMEM allocated
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(sm.tmem_slot()));

    // Dependents may be scheduled only now that this CTA holds its tensor memory: a dependent CTA that
    // shares this SM then blocks in its own allocation until this CTA has freed its columns, never the
    // other way round (it still waits for this whole grid before it reads any result).
    if (kUp) pdl_launch_dependents();

    if (a.use_pdl) pdl_wait_primary();   // up: after the row-gather kernel; down: after the gate/up kernel

    const int m_pairs = a.pair_list ? a.list_counts[0] : num_row_blocks(a) / 2;
    const int n_tiles = kUp ? a.H / 128 : (a.K + 255) / 256;
    const int num_tiles = m_pairs * n_tiles;
    const int ksteps = (kUp ? a.K : a.H) / BK;
    const int first = blockIdx.x >> 1, step = gridDim.x >> 1;   // this pair's tile sequence

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = first; t < num_tiles && ok; t += step) {
                const Coord c = tile_coord(t, m_pairs, n_tiles);
            const int pr = a.pair_list ? a.pair_list[c.m_blk] : c.m_blk;   // pair of row blocks 2*pr, 2*pr+1
                const int blk = 2 * pr + static_cast<int>(rank);
                const int e = a.expert_ids[2 * pr];
                if (leader && a.expert_ids[2 * pr + 1] != e) atomicCAS(status, 0, ST_BAD_PAIR);
                int b_row;
                if (kUp) b_row = e * a.N + c.n_tile * 128 + (leader ? 0 : a.H);
                else b_row = e * a.K + c.n_tile * 256 + static_cast<int>(rank) * 128;
                for (int ks = 0; ks < ksteps; ++ks) {
                    ok = mbar_wait_cluster(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                    if (!ok) break;
                    const uint32_t full_leader = mapa_shared(sm.full(s), 0);
                    if (leader) mbar_arrive_expect_tx(sm.full(s), 2 * PAIR_STAGE_BYTES);
                    tma_load_2d_pair(sm.a(s), &map_a, full_leader, ks * BK, blk * BM);
                    tma_load_2d_pair(sm.b(s), &map_b, full_leader, ks * BK, b_row);
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = idesc_bf16_f32(256, 256);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            bool ok = true;
            for (int t = first; t < num_tiles && ok; t += step, ++it) {
                const int buf = it & 1;
                ok = mbar_wait_cluster(sm.misc(2 + buf), ((it >> 1) & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * 256;
                for (int ks = 0; ks < ksteps; ++ks) {
                    ok = mbar_wait_cluster(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_f16_pair(d, smem_desc_sw128(sm.a(s) + k * 32), smem_desc_sw128(sm.b(s) + k * 32), idesc,
                                      (ks | k) != 0);
                    umma_commit_pair(sm.empty(s), 3);
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit_pair(sm.misc(buf), 3);
            }
        }
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const int et = threadIdx.x - 64;
        const uint32_t lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;
        const int ncg = a.epi_warps / 4;
        const int cg = ew / 4;
        if (kUp && a.zero_out) {
            int4 *o4 = reinterpret_cast<int4 *>(a.out);
            const long long n4 = static_cast<long long>(live_out_rows(a)) * a.K / 8;
            const int4 z = make_int4(0, 0, 0, 0);
            for (long long i = static_cast<long long>(blockIdx.x) * epi_threads + et; i < n4;
                 i += static_cast<long long>(gridDim.x) * epi_threads)
                o4[i] = z;
        }
        int it = 0;
        for (int t = first; t < num_tiles; t += step, ++it) {
            const Coord c = tile_coord(t, m_pairs, n_tiles);
            const int pr = a.pair_list ? a.pair_list[c.m_blk] : c.m_blk;   // pair of row blocks 2*pr, 2*pr+1
            const int blk = 2 * pr + static_cast<int>(rank);
            const int buf = it & 1;
            const uint32_t empty_leader = mapa_shared(sm.misc(2 + buf), 0);
            const uint32_t acc = tmem_base + buf * 256;
            if (kUp) {
                if (!mbar_wait(sm.misc(buf), (it >> 1) & 1, status, ST_TIMEOUT_TMEM_FULL)) break;
                if (!mbar_wait(sm.misc(5), (it & 1) ^ 1, status, ST_TIMEOUT_ACT)) break;
                tc_fence_after();
                __nv_bfloat16 *gu_row =
                    kKeep ? a.gu_out + (static_cast<size_t>(blk) * BM + row) * a.N + c.n_tile * 128 : nullptr;
                for (int ch = cg * (4 / ncg); ch < (cg + 1) * (4 / ncg); ++ch)
                    swiglu_chunk_to_smem<kKeep>(acc, lane_base, row, ch, sm.act, gu_row, a.H);
                tc_fence_before();
                mbar_arrive_cluster(empty_leader);
                fence_proxy_async_smem();
                mbar_arrive(sm.misc(4));
                if (et == 0) {
                    if (!mbar_wait(sm.misc(4), it & 1, status, ST_TIMEOUT_ACT)) break;
                    tma_store_2d(&map_act, sm.act, c.n_tile * 128, blk * BM);
                    tma_store_2d(&map_act, sm.act + ACT_TILE_BYTES / 2, c.n_tile * 128 + 64, blk * BM);
                    tma_store_commit();
                    tma_store_wait_read<0>();
                    mbar_arrive(sm.misc(5));
                }
            } else {
                const int pair = a.sorted_ids[blk * BM + row];
                const int tok = pair >= 0 ? pair / a.top_k : 0;
                const bool valid = pair >= 0 && tok < a.M;
                const float wgt = valid ? a.topk_weights[pair] : 0.f;
                const int col0 = c.n_tile * 256;
                __nv_bfloat16 *dst = valid ? out_row_ptr(a, tok, col0) : a.out;
                const int cols = min(256, a.K - col0);
                if (a.bulk_reduce && ew >= 4) break;
                if (!mbar_wait(sm.misc(buf), (it >> 1) & 1, status, ST_TIMEOUT_TMEM_FULL)) break;
                tc_fence_after();
                if (a.bulk_reduce) {
                    bulk_reduce_row(acc, lane_base, sm.act + row * RED_ROW_BYTES, wgt, dst, valid, cols, [&] {
                        tc_fence_before();
                        mbar_arrive_cluster(empty_leader);
                    });
                    continue;
                }
                for (int ch = cg * (8 / ncg); ch < (cg + 1) * (8 / ncg); ++ch)
                    reduce_chunk_to_out(tmem_addr(acc, lane_base, ch * 32), wgt, dst + ch * 32,
                                        valid && ch * 32 < cols);
                tc_fence_before();
                mbar_arrive_cluster(empty_leader);
            }
        }
        if (kUp && et == 0) tma_store_wait<0>();
        if (!kUp && a.bulk_reduce) tma_store_wait<0>();
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();      // nobody frees TMEM or exits while the peer may still use this CTA's memory
    if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
struct Problem {
    const void *x, *w, *w2;
    void *out;
    const int32_t *sorted_ids, *expert_ids, *npp;
    const float *topk_weights;
    int top_k, M, K, N, E, sorted_num, block_n, warp_n, stages, bpc, split;
};

int validate(const Problem &p, int block_m, int cpc) {
    PMOE_REQUIRE(p.x && p.w && p.w2 && p.out && p.sorted_ids && p.expert_ids && p.npp && p.topk_weights,
                 PMOE_ERR_BAD_ARG, "fused_moe_bf16: null pointer");
    PMOE_REQUIRE(p.M > 0 && p.K > 0 && p.N > 0 && p.E > 0 && p.top_k > 0 && p.sorted_num >= 0, PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16: M, K, N, num_experts, top_k must be positive");
    PMOE_REQUIRE((p.K & 127) == 0, PMOE_ERR_BAD_ARG, "K dimension must be a multiple of 128");
    PMOE_REQUIRE((p.N & 255) == 0, PMOE_ERR_BAD_ARG, "N dimension must be a multiple of 256");
    PMOE_REQUIRE((p.block_n == 64 && p.warp_n == 4) || (p.block_n == 32 && p.warp_n == 8), PMOE_ERR_UNSUPPORTED,
                 "(block_n, warp_n) must be (64, 4) or (32, 8)");
    PMOE_REQUIRE(p.stages > 0 && p.stages < 6, PMOE_ERR_UNSUPPORTED, "stages must be in 1..5");
    PMOE_REQUIRE((p.bpc == 1 || p.bpc == 2) && cpc == 1, PMOE_ERR_UNSUPPORTED,
                 "bpc must be 1 or 2 and cpc must be 1");
    PMOE_REQUIRE(p.bpc == 1 || p.split, PMOE_ERR_UNSUPPORTED, "bpc=2 (two-CTA MMA) requires split=True");
    PMOE_REQUIRE(p.bpc == 1 || p.sorted_num % 256 == 0, PMOE_ERR_BAD_ARG,
                 "bpc=2 requires routing tables built by moe_align with bpc=2 (rows padded to 256)");
    PMOE_REQUIRE(!p.split || p.stages <= 4, PMOE_ERR_UNSUPPORTED, "split=True requires stages<=4, got stages=%d",
                 p.stages);
    PMOE_REQUIRE(block_m == 128, PMOE_ERR_UNSUPPORTED, "Blackwell tcgen05 fused MoE requires block_m=128.");
    PMOE_REQUIRE(p.sorted_num % 128 == 0, PMOE_ERR_BAD_ARG, "sorted_num must be a multiple of block_m");
    PMOE_REQUIRE(static_cast<long long>(p.E) * p.N < (1ll << 31) && static_cast<long long>(p.E) * p.K < (1ll << 31),
                 PMOE_ERR_UNSUPPORTED, "E*N and E*K must fit in 31 bits");
    PMOE_REQUIRE((reinterpret_cast<uintptr_t>(p.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.w) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(p.w2) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(p.sorted_ids) & 15) == 0,
                 PMOE_ERR_BAD_ARG, "x, w, w2, out and sorted_token_ids must be 16-byte aligned");
    return PMOE_OK;
}

template <typename Kernel>
int set_smem(Kernel k, size_t bytes) {
    PMOE_CUDA_OK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
    return PMOE_OK;
}

// Byte offsets of the regions a call may carve out of its workspace. ONE function answers both "how large must
// the workspace be" and "where does the launcher put each region", whatever PMOE_PREGATHER / PMOE_AGATHER / bpc
// select at call time: every region is always reserved.
//   split != 0: activation [sorted_num, H] bf16 | x_sorted [sorted_num, K] bf16 | pair list, tail list, counts
//   split == 0: fp32 accumulation buffer [M, K] (padded to 1024 bytes) | x_sorted [sorted_num, K] bf16
struct WorkspaceLayout {
    size_t x_sorted, lists, total;
};
WorkspaceLayout plan_workspace(int M, int K, int N, int sorted_num, int split) {
    WorkspaceLayout w{};
    auto up = [](size_t v) { return (v + 1023) & ~static_cast<size_t>(1023); };
    const size_t rows = static_cast<size_t>(std::max(sorted_num, 0));
    if (!split) {
        w.x_sorted = up(static_cast<size_t>(M) * K * sizeof(float));
        w.lists = w.x_sorted + rows * K * 2;
        w.total = up(w.lists);
        return w;
    }
    w.x_sorted = rows * (N / 2) * 2;           // a multiple of 1024: sorted_num % 128 == 0 and H % 128 == 0
    w.lists = w.x_sorted + rows * K * 2;
    w.total = up(w.lists + (rows / 128 + 8) * sizeof(int32_t));   // two lists of <= blocks/2 entries + two counts
    return w;
}

// What the split launcher does with this problem under the current environment; read by run() and by the
// workspace-extent query so that the two cannot drift apart.
struct Decisions {
    int a_mode;       // gate/up A operand: 0 TMA gather4 from x, 1 row-gather pre-pass, 2 LSU gather in the kernel
    bool pregather;   // x_sorted region written and read
    bool tails;       // bpc == 2: pair / tail lists written and read
};
Decisions decide(const Problem &p) {
    Decisions d{};
    d.a_mode = a_operand_mode();
    // auto: the in-kernel LSU gather pays off when the row-gather pre-pass is a visible share of the step (its
    // cost is ~250/N of a compute-bound step) and the step is compute-bound (>= 256 routed rows per expert on
    // average; in the weight-streaming regime the pre-pass with plain tiles streams faster)
    // (TMA gather4 straight from x - 8 instead of 32 gather4 per k-step for short row blocks - was measured for
    // calls with <= 32 routed rows per expert: same time as the PDL-chained pre-pass, so it stays an option)
    if (d.a_mode < 0)
        d.a_mode = (p.bpc == 1 && p.N < 8192 && static_cast<long long>(p.M) * p.top_k >= 256ll * p.E) ? 2 : 1;
    d.pregather = d.a_mode == 1 || p.bpc == 2;   // the CTA-pair kernels always take pre-gathered rows
    d.tails = p.bpc == 2 && pair_tails_enabled();
    return d;
}

int run(const Problem &p, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    const int H = p.N / 2;
    const int max_blocks = p.sorted_num / BM;
    if (max_blocks == 0) {
        if (p.split && !call_extras().out_rows)
            PMOE_CUDA_OK(cudaMemsetAsync(p.out, 0, static_cast<size_t>(p.M) * p.K * 2, stream));
        return PMOE_OK;
    }
    Args a{};
    a.sorted_ids = p.sorted_ids;
    a.expert_ids = p.expert_ids;
    a.npp = p.npp;
    a.topk_weights = p.topk_weights;
    a.out = static_cast<__nv_bfloat16 *>(p.out);
    a.M = p.M;
    a.K = p.K;
    a.N = p.N;
    a.H = H;
    a.top_k = p.top_k;
    a.sorted_num = p.sorted_num;
    a.stages = std::min(p.stages, MAX_STAGES);
    a.epi_warps = p.warp_n;
    a.l2_ahead = l2_prefetch_distance();
    const CallExtras extras = call_extras();
    a.live_rows = extras.live_rows;
    a.out_rows = extras.out_rows;
    PMOE_REQUIRE(!extras.out_rows || p.split, PMOE_ERR_UNSUPPORTED, "fused_moe_bf16: out_rows requires split=True");
    a.gu_out = static_cast<__nv_bfloat16 *>(extras.gu_out);
    PMOE_REQUIRE(!extras.gu_out || p.split, PMOE_ERR_UNSUPPORTED,
                 "fused_moe_bf16: keeping the gate/up pre-activations requires split=True");
    const int bulk = down_bulk_reduce_mode();   // -1 auto: on when the down GEMM's K extent (H) is short
    // rows addressed through out_rows may live in a peer's memory: plain vector reductions only there
    const bool bulk_reduce = extras.out_rows ? false : (bulk < 0 ? (H <= 1024) : bulk != 0);
    const int threads = 64 + 32 * a.epi_warps;
    const int sms = sm_count();

    CUtensorMap map_x, map_w1;
    if (int rc = make_tmap_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.x, p.M, p.K, 1, BK,
                              CU_TENSOR_MAP_SWIZZLE_128B, "x"))
        return rc;
    if (int rc = make_tmap_2d(&map_w1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.w, static_cast<uint64_t>(p.E) * p.N,
                              p.K, 128, BK, CU_TENSOR_MAP_SWIZZLE_128B, "w"))
        return rc;

    if (!p.split) {
        CUtensorMap map_w2;
        if (int rc = make_tmap_2d(&map_w2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.w2,
                                  static_cast<uint64_t>(p.E) * p.K, H, 128, BK, CU_TENSOR_MAP_SWIZZLE_128B, "w2"))
            return rc;
        // workspace = fp32 accumulation buffer [M, K]: memset -> fused kernel -> out += bf16(acc32)
        PMOE_REQUIRE(workspace && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0, PMOE_ERR_BAD_ARG,
                     "fused_moe_bf16: workspace must be 16-byte aligned");
        a.acc32 = static_cast<float *>(workspace);
        const size_t elems = static_cast<size_t>(p.M) * p.K;
        const WorkspaceLayout lay = plan_workspace(p.M, p.K, p.N, p.sorted_num, 0);
        PMOE_REQUIRE(workspace_bytes >= lay.total, PMOE_ERR_BAD_ARG,
                     "fused_moe_bf16: workspace of %zu bytes required, got %zu", lay.total, workspace_bytes);
        PMOE_CUDA_OK(cudaMemsetAsync(a.acc32, 0, elems * sizeof(float), stream));
        if (pregather_enabled()) {   // x_sorted follows the accumulation buffer (1024-byte aligned)
            const size_t off = lay.x_sorted;
            __nv_bfloat16 *x_sorted = reinterpret_cast<__nv_bfloat16 *>(static_cast<uint8_t *>(workspace) + off);
            PMOE_REQUIRE((reinterpret_cast<uintptr_t>(x_sorted) & 1023) == 0, PMOE_ERR_BAD_ARG,
                         "fused_moe_bf16: workspace must be 1024-byte aligned");
            gather_rows_kernel<<<std::min(4 * sms, (p.sorted_num + 7) / 8), 256, 0, stream>>>(
                static_cast<const __nv_bfloat16 *>(p.x), x_sorted, a);
            PMOE_CUDA_OK(cudaGetLastError());
            if (int rc = make_tmap_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x_sorted, p.sorted_num, p.K, 128,
                                      BK, CU_TENSOR_MAP_SWIZZLE_128B, "x_sorted"))
                return rc;
            a.pregathered = 1;
        }
        const size_t smem = smem_bytes(a.stages, ACT_TILE_BYTES);
        if (int rc = set_smem(moe_fused_bf16_kernel, smem)) return rc;
        const int tiles = max_blocks * (H / 128);
        moe_fused_bf16_kernel<<<std::min(tiles, sms), threads, smem, stream>>>(map_x, map_w1, map_w2, a);
        PMOE_CUDA_OK(cudaGetLastError());
        const int use_pdl = pdl_enabled() ? 1 : 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(std::min<size_t>(4 * sms, (elems / 8 + 255) / 256)));
        cfg.blockDim = dim3(256);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = use_pdl ? 1 : 0;
        PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, finalize_acc32_kernel, static_cast<const float *>(a.acc32), a.out,
                                        static_cast<long long>(elems / 8), use_pdl));
        return PMOE_OK;
    }

    // split pipeline: workspace = activation [sorted_num, H] bf16 (+ x_sorted [sorted_num, K] when pre-gathering)
    PMOE_REQUIRE(workspace && (reinterpret_cast<uintptr_t>(workspace) & 1023) == 0, PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16: workspace must be 1024-byte aligned");
    const WorkspaceLayout lay = plan_workspace(p.M, p.K, p.N, p.sorted_num, 1);
    PMOE_REQUIRE(workspace_bytes >= lay.total, PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16: workspace of %zu bytes required, got %zu", lay.total, workspace_bytes);
    uint8_t *const ws_base = static_cast<uint8_t *>(workspace);
    const Decisions dec = decide(p);
    const int a_mode = dec.a_mode;
    const bool pregather = dec.pregather;
    const int phases = phase_mask();  // profiling hook: 1 = gather, 2 = gate/up, 4 = down (default all)
    if (pregather) {
        __nv_bfloat16 *x_sorted = reinterpret_cast<__nv_bfloat16 *>(ws_base + lay.x_sorted);
        if (phases & 1) {
            gather_rows_kernel<<<std::min(4 * sms, (p.sorted_num + 7) / 8), 256, 0, stream>>>(
                static_cast<const __nv_bfloat16 *>(p.x), x_sorted, a);
            PMOE_CUDA_OK(cudaGetLastError());
        }
        if (int rc = make_tmap_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x_sorted, p.sorted_num, p.K, 128, BK,
                                  CU_TENSOR_MAP_SWIZZLE_128B, "x_sorted"))
            return rc;
    }
    CUtensorMap map_act, map_w2;
    if (int rc = make_tmap_2d(&map_act, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, workspace, p.sorted_num, H, 128, BK,
                              CU_TENSOR_MAP_SWIZZLE_128B, "act"))
        return rc;
    if (int rc = make_tmap_2d(&map_w2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.w2, static_cast<uint64_t>(p.E) * p.K,
                              H, 256, BK, CU_TENSOR_MAP_SWIZZLE_128B, "w2"))
        return rc;
    CUtensorMap map_x_short = map_x, map_act_short;
    if (int rc = make_tmap_2d(&map_act_short, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, workspace, p.sorted_num, H,
                              SHORT_ROWS, BK, CU_TENSOR_MAP_SWIZZLE_128B, "act (short box)"))
        return rc;
    if (pregather)
        if (int rc = make_tmap_2d(&map_x_short, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ws_base + lay.x_sorted,
                                  p.sorted_num, p.K, SHORT_ROWS, BK, CU_TENSOR_MAP_SWIZZLE_128B, "x_sorted (short box)"))
            return rc;
    // with gu_out every row of a block is stored, so every row of the A tile must hold real data
    a.short_boxes = extras.gu_out ? 0 : short_boxes_mode();
    if (p.bpc == 2) {
        // two-CTA pipeline: always fed from the row-gathered copy; B tiles are loaded as 128-row halves
        CUtensorMap map_w2h;
        if (int rc = make_tmap_2d(&map_w2h, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.w2,
                                  static_cast<uint64_t>(p.E) * p.K, H, 128, BK, CU_TENSOR_MAP_SWIZZLE_128B, "w2"))
            return rc;
        Args pa = a;
        pa.stages = std::min(PAIR_MAX_STAGES, (a.stages * 3 + 1) / 2);   // same ring bytes as the 1-CTA kernels
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        auto launch_pair = [&](auto kernel, const CUtensorMap &ma, const CUtensorMap &mb, const Args &args, int tiles,
                               uint32_t extra, int nattr) -> int {
            const size_t smem = smem_bytes_pair(args.stages, extra);
            if (int rc = set_smem(kernel, smem)) return rc;
            PMOE_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 0));
            cudaLaunchConfig_t cfg = {};
            cfg.blockDim = dim3(threads);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = stream;
            cfg.attrs = attr;
            cfg.numAttrs = nattr;
            cfg.gridDim = dim3(2);
            int max_clusters = 0;
            PMOE_CUDA_OK(cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg));
            if (max_clusters < 1) return set_error(PMOE_ERR_CUDA, "no CTA pair of the bpc=2 kernel fits on this device");
            cfg.gridDim = dim3(2 * std::min(tiles, max_clusters));
            PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, ma, mb, map_act, args));
            return PMOE_OK;
        };
        // the last pair of an expert whose second block is empty runs as a single 128-row block on the one-CTA
        // kernels (tcgen05 does not allow cta_group::1 and ::2 in one kernel, hence own launches); PMOE_PAIR_TAILS=0
        // runs it as a pair like the others
        const bool tails = dec.tails;
        Args ta = a;    // the one-CTA launches over the tail blocks
        if (tails) {
            int32_t *lists = reinterpret_cast<int32_t *>(ws_base + lay.lists);
            const int max_pairs = max_blocks / 2;
            pa.pair_list = lists;
            pa.list_counts = lists + 2 * max_pairs;
            ta.tail_list = lists + max_pairs;
            ta.list_counts = pa.list_counts;
            ta.pregathered = 1;
            classify_pairs_kernel<<<1, 256, 0, stream>>>(p.sorted_ids, p.npp, p.sorted_num, lists, lists + max_pairs,
                                                         lists + 2 * max_pairs);
            PMOE_CUDA_OK(cudaGetLastError());
        }
        auto launch_single = [&](auto kernel, const Args &args, int tiles, size_t smem, auto... maps) -> int {
            if (int rc = set_smem(kernel, smem)) return rc;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(std::min(tiles, sms));
            cfg.blockDim = dim3(threads);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = stream;
            PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, maps..., args));
            return PMOE_OK;
        };
        if (phases & 2) {
            Args up = pa;
            up.zero_out = extras.out_rows ? 0 : 1;
            up.use_pdl = (pdl_enabled() && (phases & 1)) ? 1 : 0;
            if (int rc = a.gu_out ? launch_pair(moe_pair_bf16_kernel<true, true>, map_x, map_w1, up,
                                                (max_blocks / 2) * (H / 128), ACT_TILE_BYTES, up.use_pdl ? 2 : 1)
                                  : launch_pair(moe_pair_bf16_kernel<true>, map_x, map_w1, up,
                                                (max_blocks / 2) * (H / 128), ACT_TILE_BYTES, up.use_pdl ? 2 : 1))
                return rc;
            if (tails && !(phases & 8)) {   // plain launch: starts when the pair kernel (which zeroes `out`) has finished
                Args tu = ta;
                tu.use_pdl = 0;
                if (int rc = a.gu_out ? launch_single(moe_up_bf16_kernel<true>, tu, (max_blocks / 2) * (H / 128),
                                                      smem_bytes(tu.stages, ACT_TILE_BYTES), map_x, map_w1, map_act,
                                                      map_x_short, map_act_short)
                                      : launch_single(moe_up_bf16_kernel<false>, tu, (max_blocks / 2) * (H / 128),
                                                      smem_bytes(tu.stages, ACT_TILE_BYTES), map_x, map_w1, map_act,
                                                      map_x_short, map_act_short))
                    return rc;
            }
        }
        if (phases & 4) {
            Args dn = pa;
            dn.use_pdl = (pdl_enabled() && (phases & 2) && !tails) ? 1 : 0;
            dn.bulk_reduce = bulk_reduce ? 1 : 0;
            if (bulk_reduce) dn.stages = std::min(dn.stages, 5);   // room for the reduction staging tile
            if (int rc = launch_pair(moe_pair_bf16_kernel<false>, map_act, map_w2h, dn,
                                     (max_blocks / 2) * ((p.K + 255) / 256), bulk_reduce ? RED_STAGE_BYTES : 0u,
                                     dn.use_pdl ? 2 : 1))
                return rc;
            if (tails && !(phases & 8)) {
                Args td = ta;
                td.use_pdl = 0;
                td.down_ksplit = 1;
                td.bulk_reduce = bulk_reduce ? 1 : 0;
                if (bulk_reduce) td.stages = std::min(td.stages, 3);
                if (int rc = launch_single(moe_down_bf16_kernel, td, (max_blocks / 2) * ((p.K + 255) / 256),
                                           smem_bytes(td.stages, td.bulk_reduce ? RED_STAGE_BYTES : 0u), map_act, map_w2,
                                           map_act_short))
                    return rc;
            }
        }
        return PMOE_OK;
    }
    // two row blocks per tile (shared weight slots): PMOE_DUAL=0/1, unset = for calls with >= 1024 routed rows per
    // expert on average (measured: gate/up kernel -4..-5 % there with the in-kernel gather, -13..-15 % when fed by
    // TMA from the row-gathered copy; +5 % at 512 rows per expert, where more pairs straddle two experts)
    const int dual_env = dual_blocks_mode();
    const bool dual = a_mode != 0 && (dual_env < 0 ? static_cast<long long>(p.M) * p.top_k >= 1024ll * p.E : dual_env != 0);
    if ((phases & 2) && dual) {
        Args up = a;
        up.zero_out = extras.out_rows ? 0 : 1;
        up.pregathered = a_mode;
        up.x = static_cast<const __nv_bfloat16 *>(p.x);
        up.stages = std::min(a.stages, DUAL_MAX_STAGES);
        // LSU mode: eight gather warps (four per row block) beside four epilogue warps, else four for both blocks
        const int threads = 64 + 32 * a.epi_warps + (a_mode == 2 ? (a.epi_warps == 4 ? 2 : 1) * GATHER_THREADS : 0);
        const size_t smem = smem_bytes_dual(up.stages);
        auto dual_kernel = a.gu_out ? moe_up_dual_bf16_kernel<true> : moe_up_dual_bf16_kernel<false>;
        if (int rc = set_smem(dual_kernel, smem)) return rc;
        const int tiles = ((max_blocks + 1) / 2) * (H / 128);
        up.use_pdl = (pdl_enabled() && pregather && (phases & 1)) ? 1 : 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(std::min(tiles, sms));
        cfg.blockDim = dim3(threads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = up.use_pdl ? 1 : 0;
        PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, dual_kernel, map_x, map_w1, map_act, up));
    } else if (phases & 2) {
        Args up = a;
        up.zero_out = extras.out_rows ? 0 : 1;
        up.pregathered = a_mode;
        up.x = static_cast<const __nv_bfloat16 *>(p.x);
        const int threads = 64 + 32 * a.epi_warps + (a_mode == 2 ? GATHER_THREADS : 0);
        const size_t smem = smem_bytes(up.stages, ACT_TILE_BYTES);
        auto up_kernel = a.gu_out ? moe_up_bf16_kernel<true> : moe_up_bf16_kernel<false>;
        if (int rc = set_smem(up_kernel, smem)) return rc;
        const int tiles = max_blocks * (H / 128);
        up.use_pdl = (pdl_enabled() && pregather && (phases & 1)) ? 1 : 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(std::min(tiles, sms));
        cfg.blockDim = dim3(threads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = up.use_pdl ? 1 : 0;
        PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, up_kernel, map_x, map_w1, map_act, map_x_short, map_act_short, up));
    }
    if (phases & 4) {
        Args dn = a;
        dn.use_pdl = (pdl_enabled() && (phases & 2)) ? 1 : 0;
        dn.bulk_reduce = bulk_reduce ? 1 : 0;
        if (bulk_reduce) dn.stages = std::min(dn.stages, 3);       // room for the reduction staging tile
        const size_t smem = smem_bytes(dn.stages, dn.bulk_reduce ? RED_STAGE_BYTES : 0u);
        if (int rc = set_smem(moe_down_bf16_kernel, smem)) return rc;
        const int tiles = max_blocks * ((p.K + 255) / 256);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(std::min(tiles, sms));
        cfg.blockDim = dim3(threads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = dn.use_pdl ? 1 : 0;
        PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, moe_down_bf16_kernel, map_act, map_w2, map_act_short, dn));
    }
    return PMOE_OK;
}

}  // namespace

int wait_ns_store_bf16(unsigned long long ns) {
    PMOE_CUDA_OK(cudaMemcpyToSymbol(g_wait_ns, &ns, sizeof(ns)));
    return PMOE_OK;
}

int status_fetch_bf16(int *value, bool reset) {
    if (value) PMOE_CUDA_OK(cudaMemcpyFromSymbol(value, g_status_bf16, sizeof(int)));
    if (reset) {
        const int zero = 0;
        PMOE_CUDA_OK(cudaMemcpyToSymbol(g_status_bf16, &zero, sizeof(int)));
    }
    return PMOE_OK;
}

}  // namespace pmoe

extern "C" size_t pmoe_fused_moe_bf16_workspace_bytes(int M, int K, int N, int sorted_num, int split) {
    if (sorted_num <= 0 || N <= 0 || K <= 0 || M <= 0) return 0;
    return pmoe::plan_workspace(M, K, N, sorted_num, split).total;
}

extern "C" size_t pmoe_debug_bf16_workspace_extent(int M, int K, int N, int num_experts, int top_k, int sorted_num,
                                                   int bpc, int split) {
    using namespace pmoe;
    if (sorted_num <= 0 || N <= 0 || K <= 0 || M <= 0) return 0;
    const WorkspaceLayout lay = plan_workspace(M, K, N, sorted_num, split);
    const size_t rows = static_cast<size_t>(sorted_num);
    if (!split) return pregather_enabled() ? lay.x_sorted + rows * K * 2 : static_cast<size_t>(M) * K * sizeof(float);
    Problem p{};
    p.M = M, p.K = K, p.N = N, p.E = num_experts, p.top_k = top_k, p.sorted_num = sorted_num, p.bpc = bpc, p.split = 1;
    const Decisions d = decide(p);
    size_t end = rows * (N / 2) * 2;                                  // activation
    if (d.pregather) end = std::max(end, lay.x_sorted + rows * K * 2);
    if (d.tails) end = std::max(end, lay.lists + (2 * (rows / 256) + 2) * sizeof(int32_t));
    return end;
}

extern "C" int pmoe_fused_moe_bf16_ws(const void *x, const void *w, const void *w2, void *out,
                                      const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                      const int32_t *num_tokens_post_padded, const float *topk_weights,
                                      int top_k, int M, int K, int N, int num_experts, int sorted_num,
                                      int block_m, int block_n, int warp_n, int stages, int bpc, int cpc,
                                      int split, void *workspace, size_t workspace_bytes,
                                      pmoe_stream_t stream) {
    using namespace pmoe;
    Problem p{x, w, w2, out, sorted_token_ids, expert_ids, num_tokens_post_padded, topk_weights,
              top_k, M, K, N, num_experts, sorted_num, block_n, warp_n, stages, bpc, split ? 1 : 0};
    if (int rc = validate(p, block_m, cpc)) return rc;
    const size_t need = pmoe_fused_moe_bf16_workspace_bytes(M, K, N, sorted_num, split);
    PMOE_REQUIRE(need == 0 || (workspace && workspace_bytes >= need), PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16: workspace of %zu bytes required, got %zu", need, workspace_bytes);
    return run(p, workspace, workspace_bytes, stream);
}

extern "C" int pmoe_fused_moe_bf16(const void *x, const void *w, const void *w2, void *out,
                                   const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                   const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k,
                                   int M, int K, int N, int num_experts, int sorted_num, int block_m,
                                   int block_n, int warp_n, int stages, int bpc, int cpc, int split,
                                   pmoe_stream_t stream) {
    using namespace pmoe;
    Problem p{x, w, w2, out, sorted_token_ids, expert_ids, num_tokens_post_padded, topk_weights,
              top_k, M, K, N, num_experts, sorted_num, block_n, warp_n, stages, bpc, split ? 1 : 0};
    if (int rc = validate(p, block_m, cpc)) return rc;
    const size_t need = pmoe_fused_moe_bf16_workspace_bytes(M, K, N, sorted_num, split);
    void *raw = nullptr;
    if (need)
        if (int rc = scratch_alloc(&raw, need + 1024, stream)) return rc;
    void *ws = reinterpret_cast<void *>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int rc = run(p, raw ? ws : nullptr, need, stream);
    if (raw)
        if (int rc2 = scratch_free(raw, stream)) return rc2;
    return rc;
}

extern "C" int pmoe_fused_moe_bf16_keep_ws(const void *x, const void *w, const void *w2, void *out,
                                           const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                           const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k,
                                           int M, int K, int N, int num_experts, int sorted_num, int bpc,
                                           void *gate_up, void *workspace, size_t workspace_bytes,
                                           pmoe_stream_t stream) {
    PMOE_REQUIRE(gate_up != nullptr && (reinterpret_cast<uintptr_t>(gate_up) & 31) == 0, PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16_keep: gate_up must be a 32-byte aligned device buffer of sorted_num * N bf16");
    pmoe::CallExtras &extras = pmoe::call_extras();
    extras.gu_out = gate_up;
    const int rc = pmoe_fused_moe_bf16_ws(x, w, w2, out, sorted_token_ids, expert_ids, num_tokens_post_padded,
                                          topk_weights, top_k, M, K, N, num_experts, sorted_num, 128, 64, 4, 4, bpc, 1, 1,
                                          workspace, workspace_bytes, stream);
    extras = pmoe::CallExtras{};
    return rc;
}

extern "C" int pmoe_fused_moe_bf16_ex(const void *x, const void *w, const void *w2, void *out,
                                      const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                      const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k,
                                      int M, int K, int N, int num_experts, int sorted_num, int block_m, int block_n,
                                      int warp_n, int stages, int bpc, int cpc, int split, void *workspace,
                                      size_t workspace_bytes, const int32_t *live_rows,
                                      const unsigned long long *out_rows, pmoe_stream_t stream) {
    pmoe::CallExtras &extras = pmoe::call_extras();
    extras.live_rows = live_rows;
    extras.out_rows = out_rows;
    const int rc = pmoe_fused_moe_bf16_ws(x, w, w2, out, sorted_token_ids, expert_ids, num_tokens_post_padded,
                                          topk_weights, top_k, M, K, N, num_experts, sorted_num, block_m, block_n, warp_n,
                                          stages, bpc, cpc, split, workspace, workspace_bytes, stream);
    extras = pmoe::CallExtras{};
    return rc;
}
