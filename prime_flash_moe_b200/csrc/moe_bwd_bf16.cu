// Backward pass of the bf16 MoE FFN (the reference is forward-only, README.md:17; this is an addition).
//
// Forward, in sorted-row space (rows of sorted_token_ids, one expert per 128-row block):
//     gu   = xs @ W1[e]^T               xs = x[token(row)]            [R, N], N = 2H (gate | up)
//     act  = silu(gate) * up                                          [R, H]
//     out[token] += wt[row] * (act @ W2[e]^T)                         W2[e] is [K, H]
// Backward for d_out [T, K]:
//     d_act = wt * (dos @ W2[e])        dos = d_out[token(row)]       contraction over K, W2 read N-major
//     d_gate, d_up from d_act, gate, up (SwiGLU derivative)           d_gu [R, N]
//     d_wt[row] = sum_h (dos @ W2[e])[row, h] * act[row, h]
//     d_xs  = d_gu @ W1[e]              contraction over N, W1 read N-major; d_x[t] = sum of its rows
//     d_W2[e] = dos_e^T @ (wt * act)_e  contraction over the expert's rows, both operands M/N-major
//     d_W1[e] = d_gu_e^T @ xs_e
//
// All five contractions run on one persistent tcgen05 kernel (128 x 256 tile, K-step 64, four-slot TMA ring,
// two TMEM accumulators) whose operands are either K-major (the contraction index is contiguous in memory) or
// M/N-major (the row / column index is contiguous): the second form needs no transposed copy of anything - a
// 64 x 64 TMA box of the row-major tensor lands in shared memory as eight 8-row swizzle atoms, which is the
// canonical M/N-major 128-byte-swizzle operand layout (atom stride along K = 1024 B, along M/N = the box size).
//
// Algorithmic bytes (one pass each): weights 2 x (read W1, W2; write dW1, dW2) and the row-space intermediates
// xs, dos, gu, d_gu, act [R, K | N | H]; FLOPs = 3 x forward (gu recompute + 2 dgrad + 2 wgrad = 5 GEMMs of the
// forward's two sizes: 2*R*K*N x 3 + 2*R*K*H x 2).
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

#include "host_common.h"
#include "ptx.cuh"
#include "tile_sched.cuh"

namespace pmoe {

__device__ int g_status_bwd = 0;

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr uint32_t BOX_BYTES = 64 * 64 * 2;           // one 64 x 64 bf16 box: 8 KB, eight swizzle atoms
constexpr uint32_t A_BYTES = BM * BK * 2;             // 16 KB
constexpr uint32_t B_BYTES = BN * BK * 2;             // 32 KB
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;   // 48 KB
constexpr int STAGES = 4;
constexpr uint32_t TMEM_COLS = 512;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + EPI_WARPS * 32;
constexpr size_t SMEM_BYTES = 1024 + static_cast<size_t>(STAGES) * STAGE_BYTES + 256;

enum : int {
    MODE_NT_STORE = 0,     // C[R, n] = A[R, k] . B[e][n, k]^T          A, B K-major       plain bf16 store
    MODE_NN_SWIGLU = 1,    // C[R, h] = A[R, k] . B[e][k, h]            B N-major          SwiGLU backward epilogue
    MODE_NN_STORE = 2,     // C[R, n] = A[R, k] . B[e][k, n]            B N-major          plain bf16 store
    MODE_WGRAD = 3,        // C[e][m, n] = sum over the expert's rows A[r, m] . B[r, n]    both M/N-major
    MODE_WGRAD_X = 4,      // the same with an fp32 and / or accumulated gradient (C = or += per GArgs::c_f32, accumulate)
};
__host__ __device__ constexpr bool is_wgrad(int mode) { return mode >= MODE_WGRAD; }

struct GArgs {
    int mode;
    const int32_t *sorted_ids, *expert_ids, *npp;
    int sorted_num;
    const int32_t *eblk;          // MODE_WGRAD: first / one-past-last row block of every expert, [2 * E]
    const int32_t *items;         // row-space modes: the row blocks of this launch (pair kernel: first block of each
    const int32_t *item_count;    //   pair) and their number on the device; null = every live row block
    const float *topk_weights;
    int top_k, tokens, E;
    int ksteps;                   // modes 0-2: contraction length / 64
    int n_tiles;                  // 256-column tiles of C
    int m_tiles;                  // MODE_WGRAD: 128-row tiles of one expert's C
    int b_rows_per_expert;        // rows of one expert in B's 2-D view (modes 0-2)
    __nv_bfloat16 *c;
    long long ldc;
    int c_cols;                   // live columns of C
    int c_rows;                   // MODE_WGRAD: rows of one expert's C
    float *c_f32;                 // MODE_WGRAD_X: fp32 gradient (then `c` is unused), else null
    int accumulate;               // MODE_WGRAD_X: add to the gradient already there instead of overwriting it
    // MODE_NN_SWIGLU
    const __nv_bfloat16 *gu;      // [R, N] gate | up pre-activations
    __nv_bfloat16 *dgu;           // [R, N]
    __nv_bfloat16 *actw;          // [R, H] wt * silu(gate) * up
    float *dwt;                   // [tokens * top_k] or null
    int H, N;
};

// ---------------------------------------------------------------------------------------------
// row-space helpers (HBM-bound)
// ---------------------------------------------------------------------------------------------
// xs[r] = x[token(r)] and dos[r] = d_out[token(r)] for the live rows, zeros for padding rows. One warp per row,
// both tensors in one pass over the routing table; kWide: 32 bytes per lane and access (x and d_out 32-byte
// aligned), else 16.
template <bool kWide>
__global__ void __launch_bounds__(256)
gather_token_rows_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ d_out,
                         const int32_t *__restrict__ sorted_ids, const int32_t *__restrict__ npp, int sorted_num,
                         int top_k, int tokens, int K, __nv_bfloat16 *__restrict__ xs, __nv_bfloat16 *__restrict__ dos) {
    const int rows = live_row_blocks(npp, sorted_num) * BM;
    const int lane = threadIdx.x & 31;
    constexpr int kElems = kWide ? 16 : 8;        // bf16 per lane and access
    const int vec_per_row = K / kElems;
    for (int r = blockIdx.x * 8 + (threadIdx.x >> 5); r < rows; r += gridDim.x * 8) {
        const int pair = sorted_ids[r];
        const int tok = pair >= 0 ? pair / top_k : tokens;
        const bool live = tok < tokens;
        const __nv_bfloat16 *s1 = x + static_cast<size_t>(live ? tok : 0) * K;
        const __nv_bfloat16 *s2 = d_out + static_cast<size_t>(live ? tok : 0) * K;
        __nv_bfloat16 *d1 = xs + static_cast<size_t>(r) * K;
        __nv_bfloat16 *d2 = dos + static_cast<size_t>(r) * K;
#pragma unroll 4
        for (int v = lane; v < vec_per_row; v += 32) {
            if (kWide) {
                uint32_t a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                if (live) {
                    ld_global_v8(s1 + v * 16, a);
                    ld_global_v8(s2 + v * 16, b);
                }
                st_global_v8(d1 + v * 16, a);
                st_global_v8(d2 + v * 16, b);
            } else {
                uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
                if (live) {
                    a = __ldg(reinterpret_cast<const uint4 *>(s1) + v);
                    b = __ldg(reinterpret_cast<const uint4 *>(s2) + v);
                }
                reinterpret_cast<uint4 *>(d1)[v] = a;
                reinterpret_cast<uint4 *>(d2)[v] = b;
            }
        }
    }
}

// inv[pair] = sorted row of the pair (inv is preset to -1); eblk[e] / eblk[E + e] = range of the blocks of expert e
// that hold routed rows (preset to 0)
__global__ void __launch_bounds__(256)
row_maps_kernel(const int32_t *__restrict__ sorted_ids, const int32_t *__restrict__ expert_ids,
                const int32_t *__restrict__ npp, int sorted_num, int top_k, int tokens, int E,
                int32_t *__restrict__ inv, int32_t *__restrict__ eblk) {
    const int blocks = live_row_blocks(npp, sorted_num);
    const int rows = blocks * BM;
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
        const int pair = sorted_ids[r];
        if (pair >= 0 && pair < tokens * top_k) inv[pair] = r;
        if ((r & (BM - 1)) == 0) {
            // routed rows come first in an expert's segment, so a block is live iff its first row is; routing
            // tables padded to 256 rows (bpc = 2) can end an expert with one block without any routed row
            const int b = r / BM, e = expert_ids[b];
            if (e >= 0 && e < E && pair >= 0) {
                if (b == 0 || expert_ids[b - 1] != e) eblk[e] = b;
                const bool more = b + 1 < blocks && expert_ids[b + 1] == e && sorted_ids[(b + 1) * BM] >= 0;
                if (!more) eblk[E + e] = b + 1;
            }
        }
    }
}

// dx[t] = sum over the token's top_k routes of d_xs[row of the route] (fp32 sum, one rounding)
__global__ void __launch_bounds__(256)
combine_dx_kernel(const __nv_bfloat16 *__restrict__ dxs, const int32_t *__restrict__ inv, int top_k, int tokens,
                  int K, __nv_bfloat16 *__restrict__ dx) {
    const int vec_per_row = K / 8;
    const long long total = static_cast<long long>(tokens) * vec_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(i / vec_per_row), v = static_cast<int>(i - static_cast<long long>(t) * vec_per_row);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < top_k; ++j) {
            const int r = inv[t * top_k + j];
            if (r < 0) continue;
            const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(dxs + static_cast<size_t>(r) * K) + v);
            const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc[2 * q] += __low2float(h[q]);
                acc[2 * q + 1] += __high2float(h[q]);
            }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        reinterpret_cast<uint4 *>(dx + static_cast<size_t>(t) * K)[v] = o;
    }
}

// ---------------------------------------------------------------------------------------------
// the grouped GEMM
//   warp 0: TMA producer | warp 1: TMEM owner + MMA issuer | warps 2-9: epilogue (lane quarter = warp % 4,
//   column half = (warp - 2) / 4)
//   misc barriers: 0,1 tmem_full[2] | 2,3 tmem_empty[2]
// ---------------------------------------------------------------------------------------------
struct Ring {
    uint32_t ring, bars;
    __device__ __forceinline__ uint32_t a(int s) const { return ring + s * STAGE_BYTES; }
    __device__ __forceinline__ uint32_t b(int s) const { return ring + s * STAGE_BYTES + A_BYTES; }
    __device__ __forceinline__ uint32_t full(int s) const { return bars + 8 * s; }
    __device__ __forceinline__ uint32_t empty(int s) const { return bars + 8 * (STAGES + s); }
    __device__ __forceinline__ uint32_t misc(int i) const { return bars + 8 * (2 * STAGES + i); }
    __device__ __forceinline__ uint32_t tmem_slot() const { return bars + 8 * (2 * STAGES + 4); }
};

// Shared-memory descriptor of an M/N-major operand made of 64 x 64 boxes written by TMA with SWIZZLE_128B: one
// 128-byte line holds 64 consecutive M (or N) indices of one k, eight lines (8 k) form a 1024-byte swizzle atom;
// atoms follow each other along k every 1024 B (stride byte offset) and along M/N every box (leading byte offset).
// Stepping by one MMA (16 k) adds 2048 B to `addr`.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(BOX_BYTES >> 4) << 16) |
           (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

struct Tile {
    int mb, nt, e, mt, k0, k1;
};

// row-space modes: the row blocks of this launch are either all live ones or those named by a.items
__device__ __forceinline__ int num_row_items(const GArgs &a) {
    return a.items ? *a.item_count : live_row_blocks(a.npp, a.sorted_num);
}

template <int MODE>
__device__ __forceinline__ Tile decode_tile(const GArgs &a, int t, int m_items) {
    Tile tl;
    if (is_wgrad(MODE)) {
        const int per = a.m_tiles * a.n_tiles;
        tl.e = t / per;
        const int rem = t - tl.e * per;
        tl.mt = rem % a.m_tiles;
        tl.nt = rem / a.m_tiles;
        tl.mb = 0;
        tl.k0 = 2 * a.eblk[tl.e];              // k-step = 64-row chunk of the sorted row space
        tl.k1 = 2 * a.eblk[a.E + tl.e];
    } else {
        const Coord c = tile_coord(t, m_items, a.n_tiles);
        tl.mb = a.items ? a.items[c.m_blk] : c.m_blk;
        tl.nt = c.n_tile;
        tl.mt = 0;
        tl.e = max(0, min(a.E - 1, a.expert_ids[tl.mb]));
        tl.k0 = 0;
        tl.k1 = a.sorted_ids[tl.mb * BM] >= 0 ? a.ksteps : 0;    // a block without routed rows is skipped altogether
    }
    return tl;
}

// 32 fp32 -> 32 bf16 = 64 contiguous bytes as two 256-bit stores (every store fills a whole 32-byte sector, so a
// warp whose lanes hold different rows still writes full sectors); `dst` must be 32-byte aligned
__device__ __forceinline__ void store_chunk_bf16(__nv_bfloat16 *dst, const float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        uint32_t w[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) w[q] = pack_bf16x2(v[16 * j + 2 * q], v[16 * j + 2 * q + 1]);
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 16 * j), "r"(w[0]), "r"(w[1]),
                     "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                     : "memory");
    }
}

__device__ __forceinline__ void load_chunk_bf16(const __nv_bfloat16 *src, float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        uint32_t w[8];
        asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                     : "l"(src + 16 * j));
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            v[16 * j + 2 * q] = __uint_as_float(w[q] << 16);
            v[16 * j + 2 * q + 1] = __uint_as_float(w[q] & 0xffff0000u);
        }
    }
}



// Epilogue of one finished accumulator (128 rows x 256 columns at TMEM `acc`), shared by both GEMM kernels: thread
// = row `row` of the accumulator, column chunks cg*4 .. cg*4+3 (32 columns each). Row-space modes: `mb` = row
// block; MODE_WGRAD: `m` = row of the expert's gradient matrix.
template <int MODE>
__device__ __forceinline__ void drain_tile(const GArgs &a, uint32_t acc, uint32_t lane_base, int row, int cg, int mb,
                                           int e, int m, int col0) {
    if (MODE == MODE_NN_SWIGLU) {
        const size_t row_g = static_cast<size_t>(mb) * BM + row;
        const int pair = a.sorted_ids[row_g];
        const bool valid = pair >= 0 && pair < a.tokens * a.top_k;
        const float wt = valid ? a.topk_weights[pair] : 0.f;
        float part = 0.f;
        for (int ch = cg * 4; ch < cg * 4 + 4; ++ch) {
            const int h0 = col0 + ch * 32;
            if (h0 >= a.H) break;
            float c[32], g[32], u[32];
            tmem_ld_32x32(c, tmem_addr(acc, lane_base, ch * 32));
            load_chunk_bf16(a.gu + row_g * a.N + h0, g);
            load_chunk_bf16(a.gu + row_g * a.N + a.H + h0, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float s = 1.f / (1.f + __expf(-g[j]));
                const float silu = g[j] * s;
                const float act = silu * u[j];
                const float d = wt * c[j];
                part += c[j] * act;
                c[j] = wt * act;                                   // -> actw
                g[j] = d * u[j] * s * (1.f + g[j] * (1.f - s));    // -> d_gate
                u[j] = d * silu;                                   // -> d_up
            }
            store_chunk_bf16(a.actw + row_g * a.H + h0, c);
            store_chunk_bf16(a.dgu + row_g * a.N + h0, g);
            store_chunk_bf16(a.dgu + row_g * a.N + a.H + h0, u);
        }
        if (a.dwt && valid) atomicAdd(a.dwt + pair, part);
        return;
    }
    if (MODE == MODE_WGRAD_X) {
        // fp32 and / or accumulated weight gradient: a lane owns 32 consecutive columns of its row per chunk
        if (m >= a.c_rows) return;
        const size_t off = (static_cast<size_t>(e) * a.c_rows + m) * a.ldc + col0;
        for (int ch = cg * 4; ch < cg * 4 + 4; ++ch) {
            if (col0 + ch * 32 >= a.c_cols) break;
            float v[32], old[32];
            tmem_ld_32x32(v, tmem_addr(acc, lane_base, ch * 32));
            if (a.accumulate) {
                if (a.c_f32) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t w[8];
                        ld_global_v8(a.c_f32 + off + ch * 32 + 8 * j, w);
#pragma unroll
                        for (int q = 0; q < 8; ++q) old[8 * j + q] = __uint_as_float(w[q]);
                    }
                } else {
                    load_chunk_bf16(a.c + off + ch * 32, old);
                }
            }
            tmem_ld_wait();
            if (a.accumulate) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += old[j];
            }
            if (a.c_f32) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t w[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) w[q] = __float_as_uint(v[8 * j + q]);
                    st_global_v8(a.c_f32 + off + ch * 32 + 8 * j, w);
                }
            } else {
                store_chunk_bf16(a.c + off + ch * 32, v);
            }
        }
        return;
    }
    __nv_bfloat16 *dst;
    bool row_ok = true;
    if (MODE == MODE_WGRAD) {
        row_ok = m < a.c_rows;
        dst = a.c + (static_cast<size_t>(e) * a.c_rows + (row_ok ? m : 0)) * a.ldc + col0;
    } else {
        dst = a.c + (static_cast<size_t>(mb) * BM + row) * a.ldc + col0;
    }
    for (int ch = cg * 4; ch < cg * 4 + 4; ++ch) {
        if (col0 + ch * 32 >= a.c_cols) break;
        float v[32];
        tmem_ld_32x32(v, tmem_addr(acc, lane_base, ch * 32));
        tmem_ld_wait();
        if (row_ok) store_chunk_bf16(dst + ch * 32, v);
    }
}

// MODE_WGRAD, an expert without rows: its weight gradient is zero (no accumulator involved)
__device__ __forceinline__ void zero_tile(const GArgs &a, int cg, int e, int m, int col0) {
    if (m >= a.c_rows || a.accumulate) return;      // nothing to add
    if (a.c_f32) {
        float *dst32 = a.c_f32 + (static_cast<size_t>(e) * a.c_rows + m) * a.ldc + col0;
        for (int ch = cg * 4; ch < cg * 4 + 4; ++ch)
            if (col0 + ch * 32 < a.c_cols)
                for (int j = 0; j < 8; ++j) reinterpret_cast<uint4 *>(dst32 + ch * 32)[j] = make_uint4(0, 0, 0, 0);
        return;
    }
    __nv_bfloat16 *dst = a.c + (static_cast<size_t>(e) * a.c_rows + m) * a.ldc + col0;
    for (int ch = cg * 4; ch < cg * 4 + 4; ++ch)
        if (col0 + ch * 32 < a.c_cols)
            for (int j = 0; j < 4; ++j) reinterpret_cast<uint4 *>(dst + ch * 32)[j] = make_uint4(0, 0, 0, 0);
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
moe_bwd_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GArgs a) {
    extern __shared__ uint8_t smem_raw[];
    Ring sm;
    sm.ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    sm.bars = sm.ring + STAGES * STAGE_BYTES;
    int *status = &g_status_bwd;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        mbar_init(sm.misc(0), 1);
        mbar_init(sm.misc(1), 1);
        mbar_init(sm.misc(2), EPI_WARPS * 32);
        mbar_init(sm.misc(3), EPI_WARPS * 32);
        fence_mbar_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if (warp == 1) tmem_alloc(sm.tmem_slot(), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(sm.tmem_slot()));

    constexpr bool a_mn = is_wgrad(MODE);
    constexpr bool b_mn = MODE != MODE_NT_STORE;
    const int m_items = a_mn ? 0 : num_row_items(a);
    const int num_tiles = a_mn ? a.E * a.m_tiles * a.n_tiles : m_items * a.n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            long long issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const Tile tl = decode_tile<MODE>(a, t, m_items);
                for (int ks = tl.k0; ks < tl.k1; ++ks) {
                    ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_arrive_expect_tx(sm.full(s), STAGE_BYTES);
                    if (a_mn) {
#pragma unroll
                        for (int i = 0; i < 2; ++i)
                            tma_load_2d(sm.a(s) + i * BOX_BYTES, &map_a, sm.full(s), tl.mt * BM + i * 64, ks * 64);
                    } else {
                        tma_load_2d(sm.a(s), &map_a, sm.full(s), ks * BK, tl.mb * BM);
                    }
                    if (!b_mn) {
                        tma_load_2d(sm.b(s), &map_b, sm.full(s), ks * BK, tl.e * a.b_rows_per_expert + tl.nt * BN);
                    } else {
                        const int krow = a_mn ? ks * 64 : tl.e * a.b_rows_per_expert + ks * 64;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            tma_load_2d(sm.b(s) + j * BOX_BYTES, &map_b, sm.full(s), tl.nt * BN + j * 64, krow);
                    }
                    ++issued;
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
            if (!ok) {
                // give the copies already issued a bounded time to land before the CTA exits
                const long long first = issued > STAGES ? issued - STAGES : 0;
                for (long long f = first; f < issued; ++f) {
                    const uint32_t bar = sm.full(static_cast<int>(f % STAGES));
                    const uint32_t parity = static_cast<uint32_t>((f / STAGES) & 1);
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(bar, parity))
                        if (globaltimer_ns() - t0 > 20000000ull) break;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(BM, BN) | (a_mn ? 1u << 15 : 0u) | (b_mn ? 1u << 16 : 0u);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const Tile tl = decode_tile<MODE>(a, t, m_items);
                if (tl.k1 <= tl.k0) continue;
                const int buf = it & 1;
                ok = mbar_wait(sm.misc(2 + buf), ((it >> 1) & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * BN;
                for (int ks = tl.k0; ks < tl.k1; ++ks) {
                    ok = mbar_wait(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = a_mn ? smem_desc_mn_sw128(sm.a(s) + k * 2048) : smem_desc_sw128(sm.a(s) + k * 32);
                        const uint64_t bd = b_mn ? smem_desc_mn_sw128(sm.b(s) + k * 2048) : smem_desc_sw128(sm.b(s) + k * 32);
                        umma_f16(d, ad, bd, idesc, (ks != tl.k0) || (k != 0));
                    }
                    umma_commit(sm.empty(s));
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit(sm.misc(buf));
                ++it;
            }
        }
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const uint32_t lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;
        const int cg = ew / 4;
        int it = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
            const Tile tl = decode_tile<MODE>(a, t, m_items);
            const int col0 = tl.nt * BN;
            const int m = tl.mt * BM + row;
            if (tl.k1 <= tl.k0) {
                if (a_mn) zero_tile(a, cg, tl.e, m, col0);
                continue;
            }
            const int buf = it & 1;
            if (!mbar_wait(sm.misc(buf), (it >> 1) & 1, status, ST_TIMEOUT_TMEM_FULL)) break;
            tc_fence_after();
            drain_tile<MODE>(a, tmem_base + buf * BN, lane_base, row, cg, tl.mb, tl.e, m, col0);
            tc_fence_before();
            mbar_arrive(sm.misc(2 + buf));
            ++it;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// The same GEMMs on CTA pairs (cluster of 2, tcgen05 cta_group::2, M = 256). Row-space modes: the pair takes two
// row blocks of one expert (a.items lists the first block of every such pair; the odd last block of an expert goes
// to the one-CTA kernel). MODE_WGRAD: 256 rows of the expert's gradient matrix. Each CTA loads its own 128 rows /
// M indices of A and its own 128 of the tile's 256 N indices of B: 32 KB per ring slot and CTA instead of 48 KB
// (six slots), the even CTA issues the MMAs for both, each CTA drains the accumulator rows of its half. No
// multicast loads; ring slots and accumulators are released to both CTAs by multicast tcgen05.commit.
//   misc barriers: 0,1 tmem_full[2] | 2,3 tmem_empty[2] (even CTA; both CTAs' epilogue warps arrive there)
// ---------------------------------------------------------------------------------------------
constexpr uint32_t PAIR_STAGE_BYTES = 4 * BOX_BYTES;   // 32 KB
constexpr int PAIR_STAGES = 6;
constexpr size_t PAIR_SMEM_BYTES = 1024 + static_cast<size_t>(PAIR_STAGES) * PAIR_STAGE_BYTES + 256;

struct RingPair {
    uint32_t ring, bars;
    __device__ __forceinline__ uint32_t a(int s) const { return ring + s * PAIR_STAGE_BYTES; }
    __device__ __forceinline__ uint32_t b(int s) const { return ring + s * PAIR_STAGE_BYTES + 2 * BOX_BYTES; }
    __device__ __forceinline__ uint32_t full(int s) const { return bars + 8 * s; }
    __device__ __forceinline__ uint32_t empty(int s) const { return bars + 8 * (PAIR_STAGES + s); }
    __device__ __forceinline__ uint32_t misc(int i) const { return bars + 8 * (2 * PAIR_STAGES + i); }
    __device__ __forceinline__ uint32_t tmem_slot() const { return bars + 8 * (2 * PAIR_STAGES + 4); }
};

// tile of a pair: row-space modes mb = first row block of the pair; MODE_WGRAD mt = 256-row tile of the gradient
template <int MODE>
__device__ __forceinline__ Tile decode_pair_tile(const GArgs &a, int t, int m_items, int m_tiles2) {
    Tile tl;
    if (is_wgrad(MODE)) {
        const int per = m_tiles2 * a.n_tiles;
        tl.e = t / per;
        const int rem = t - tl.e * per;
        tl.mt = rem % m_tiles2;
        tl.nt = rem / m_tiles2;
        tl.mb = 0;
        tl.k0 = 2 * a.eblk[tl.e];
        tl.k1 = 2 * a.eblk[a.E + tl.e];
    } else {
        const Coord c = tile_coord(t, m_items, a.n_tiles);
        tl.mb = a.items[c.m_blk];
        tl.nt = c.n_tile;
        tl.mt = 0;
        tl.e = max(0, min(a.E - 1, a.expert_ids[tl.mb]));
        tl.k0 = 0;
        tl.k1 = a.ksteps;
    }
    return tl;
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
moe_bwd_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GArgs a) {
    extern __shared__ uint8_t smem_raw[];
    RingPair sm;
    sm.ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    sm.bars = sm.ring + PAIR_STAGES * PAIR_STAGE_BYTES;
    int *status = &g_status_bwd;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        mbar_init(sm.misc(0), 1);
        mbar_init(sm.misc(1), 1);
        mbar_init(sm.misc(2), 2 * EPI_WARPS * 32);
        mbar_init(sm.misc(3), 2 * EPI_WARPS * 32);
        fence_mbar_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if (warp == 1) tmem_alloc_pair(sm.tmem_slot(), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();      // both CTAs' barriers are initialised and both halves of TMEM allocated
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(sm.tmem_slot()));

    constexpr bool wgrad = is_wgrad(MODE);
    constexpr bool b_mn = MODE != MODE_NT_STORE;
    const int m_tiles2 = (a.c_rows + 255) / 256;
    const int m_items = wgrad ? 0 : *a.item_count;
    const int num_tiles = wgrad ? a.E * m_tiles2 * a.n_tiles : m_items * a.n_tiles;
    const int first = blockIdx.x >> 1, step = gridDim.x >> 1;   // this pair's tile sequence

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = first; t < num_tiles && ok; t += step) {
                const Tile tl = decode_pair_tile<MODE>(a, t, m_items, m_tiles2);
                const int m0 = tl.mt * 256 + static_cast<int>(rank) * 128;      // wgrad: this CTA's M indices
                const int blk = tl.mb + static_cast<int>(rank);                 // row space: this CTA's row block
                const int n0 = tl.nt * BN + static_cast<int>(rank) * 128;       // this CTA's N indices of B
                for (int ks = tl.k0; ks < tl.k1; ++ks) {
                    ok = mbar_wait_cluster(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                    if (!ok) break;
                    const uint32_t full_leader = mapa_shared(sm.full(s), 0);
                    if (leader) mbar_arrive_expect_tx(sm.full(s), 2 * PAIR_STAGE_BYTES);
                    if (wgrad) {
#pragma unroll
                        for (int i = 0; i < 2; ++i)
                            tma_load_2d_pair(sm.a(s) + i * BOX_BYTES, &map_a, full_leader, m0 + i * 64, ks * 64);
                    } else {
                        tma_load_2d_pair(sm.a(s), &map_a, full_leader, ks * BK, blk * BM);
                    }
                    if (!b_mn) {
                        tma_load_2d_pair(sm.b(s), &map_b, full_leader, ks * BK, tl.e * a.b_rows_per_expert + n0);
                    } else {
                        const int krow = wgrad ? ks * 64 : tl.e * a.b_rows_per_expert + ks * 64;
#pragma unroll
                        for (int j = 0; j < 2; ++j)
                            tma_load_2d_pair(sm.b(s) + j * BOX_BYTES, &map_b, full_leader, n0 + j * 64, krow);
                    }
                    if (++s == PAIR_STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = idesc_bf16_f32(256, 256) | (wgrad ? 1u << 15 : 0u) | (b_mn ? 1u << 16 : 0u);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            bool ok = true;
            for (int t = first; t < num_tiles && ok; t += step) {
                const Tile tl = decode_pair_tile<MODE>(a, t, m_items, m_tiles2);
                if (tl.k1 <= tl.k0) continue;
                const int buf = it & 1;
                ok = mbar_wait_cluster(sm.misc(2 + buf), ((it >> 1) & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * BN;
                for (int ks = tl.k0; ks < tl.k1; ++ks) {
                    ok = mbar_wait_cluster(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = wgrad ? smem_desc_mn_sw128(sm.a(s) + k * 2048) : smem_desc_sw128(sm.a(s) + k * 32);
                        const uint64_t bd = b_mn ? smem_desc_mn_sw128(sm.b(s) + k * 2048) : smem_desc_sw128(sm.b(s) + k * 32);
                        umma_f16_pair(d, ad, bd, idesc, (ks != tl.k0) || (k != 0));
                    }
                    umma_commit_pair(sm.empty(s), 3);
                    if (++s == PAIR_STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit_pair(sm.misc(buf), 3);
                ++it;
            }
        }
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const uint32_t lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;
        const int cg = ew / 4;
        int it = 0;
        for (int t = first; t < num_tiles; t += step) {
            const Tile tl = decode_pair_tile<MODE>(a, t, m_items, m_tiles2);
            const int col0 = tl.nt * BN;
            const int m = tl.mt * 256 + static_cast<int>(rank) * 128 + row;
            if (tl.k1 <= tl.k0) {
                if (wgrad) zero_tile(a, cg, tl.e, m, col0);
                continue;
            }
            const int buf = it & 1;
            if (!mbar_wait(sm.misc(buf), (it >> 1) & 1, status, ST_TIMEOUT_TMEM_FULL)) break;
            tc_fence_after();
            drain_tile<MODE>(a, tmem_base + buf * BN, lane_base, row, cg, tl.mb + static_cast<int>(rank), tl.e, m, col0);
            tc_fence_before();
            mbar_arrive_cluster(mapa_shared(sm.misc(2 + buf), 0));
            ++it;
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();      // nobody frees TMEM or exits while the peer may still use this CTA's memory
    if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// The row blocks that hold routed rows, in order, one CTA: live_list[0 .. *live_count). The row-space GEMMs walk this
// list, so that blocks without routed rows (routing tables padded to 256 rows) cost no tile slot in the static
// schedule.
__global__ void __launch_bounds__(1024)
live_items_kernel(const int32_t *__restrict__ eblk, int E, int32_t *__restrict__ live_list,
                  int32_t *__restrict__ live_count) {
    __shared__ int sn[1024];
    const int e = threadIdx.x;
    const int b0 = e < E ? eblk[e] : 0;
    const int nb = e < E ? max(0, eblk[E + e] - b0) : 0;
    sn[e] = nb;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {
        const int v = e >= d ? sn[e - d] : 0;
        __syncthreads();
        sn[e] += v;
        __syncthreads();
    }
    const int off = sn[e] - nb;
    for (int j = 0; j < nb; ++j) live_list[off + j] = b0 + j;
    if (e == 1023) *live_count = sn[e];
}

// Work lists of the row-space GEMMs on CTA pairs, one CTA: for every expert its row blocks two by two (pair_list =
// first block of each pair) and the odd last one (single_list); counts[0] = pairs, counts[1] = singles.
__global__ void __launch_bounds__(1024)
pair_items_kernel(const int32_t *__restrict__ eblk, int E, int32_t *__restrict__ pair_list,
                  int32_t *__restrict__ single_list, int32_t *__restrict__ counts) {
    __shared__ int sp[1024], ss[1024];
    const int e = threadIdx.x;
    const int b0 = e < E ? eblk[e] : 0;
    const int nb = e < E ? max(0, eblk[E + e] - b0) : 0;
    sp[e] = nb / 2;
    ss[e] = nb & 1;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {      // inclusive scans of both counts
        const int vp = e >= d ? sp[e - d] : 0, vs = e >= d ? ss[e - d] : 0;
        __syncthreads();
        sp[e] += vp;
        ss[e] += vs;
        __syncthreads();
    }
    const int poff = sp[e] - nb / 2, soff = ss[e] - (nb & 1);
    for (int j = 0; j < nb / 2; ++j) pair_list[poff + j] = b0 + 2 * j;
    if (nb & 1) single_list[soff] = b0 + nb - 1;
    if (e == 1023) {
        counts[0] = sp[e];
        counts[1] = ss[e];
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------------------------
namespace {

size_t align_up(size_t v) { return (v + 1023) & ~static_cast<size_t>(1023); }

struct BwdLayout {
    size_t xs, dos, gu, dgu, actw, inv, eblk, pair_list, single_list, counts, live_list, total;
};

// xs | dos (reused for d_xs once dW2 is done) | gu | d_gu | wt*act | pair -> row | expert block ranges | work lists
BwdLayout plan_backward(int T, int K, int N, int E, int top_k, int sorted_num) {
    const size_t R = static_cast<size_t>(sorted_num);
    BwdLayout l{};
    size_t off = 0;
    l.xs = off, off = align_up(off + R * K * 2);
    l.dos = off, off = align_up(off + R * K * 2);
    l.gu = off, off = align_up(off + R * N * 2);
    l.dgu = off, off = align_up(off + R * N * 2);
    l.actw = off, off = align_up(off + R * (N / 2) * 2);
    l.inv = off, off = align_up(off + static_cast<size_t>(T) * top_k * sizeof(int32_t));
    l.eblk = off, off = align_up(off + 2 * static_cast<size_t>(E) * sizeof(int32_t));
    l.pair_list = off, off = align_up(off + (R / 256 + 1) * sizeof(int32_t));
    l.single_list = off, off = align_up(off + static_cast<size_t>(E) * sizeof(int32_t));
    l.counts = off, off = align_up(off + 3 * sizeof(int32_t));            // pairs, singles, live blocks
    l.live_list = off, off = align_up(off + (R / 128 + 1) * sizeof(int32_t));
    l.total = off;
    return l;
}

template <int MODE>
int launch_gemm_mode(const CUtensorMap &ma, const CUtensorMap &mb, const GArgs &g, cudaStream_t stream) {
    static bool configured[64] = {false};
    int dev = 0;
    PMOE_CUDA_OK(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        PMOE_CUDA_OK(cudaFuncSetAttribute(moe_bwd_gemm_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(SMEM_BYTES)));
        configured[dev] = true;
    }
    moe_bwd_gemm_kernel<MODE><<<sm_count(), THREADS, SMEM_BYTES, stream>>>(ma, mb, g);
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}

int launch_gemm(const CUtensorMap &ma, const CUtensorMap &mb, const GArgs &g, cudaStream_t stream) {
    switch (g.mode) {
        case MODE_NT_STORE: return launch_gemm_mode<MODE_NT_STORE>(ma, mb, g, stream);
        case MODE_NN_SWIGLU: return launch_gemm_mode<MODE_NN_SWIGLU>(ma, mb, g, stream);
        case MODE_NN_STORE: return launch_gemm_mode<MODE_NN_STORE>(ma, mb, g, stream);
        case MODE_WGRAD: return launch_gemm_mode<MODE_WGRAD>(ma, mb, g, stream);
        default: return launch_gemm_mode<MODE_WGRAD_X>(ma, mb, g, stream);
    }
}

// PMOE_BWD_PAIRS: 0 = one-CTA kernel everywhere; 1 = weight-gradient GEMMs on CTA pairs; 2 = the row-space GEMMs as
// well (measured: no gain, their odd-last-block launch eats it); unset (-1) = 1 when an expert has 256 routed rows or
// more on average (below that the weight-gradient launches are bound by their stores and the pairs measured slower)
int pairs_mode() {
    const char *v = getenv("PMOE_BWD_PAIRS");
    return (v && v[0] >= '0' && v[0] <= '2') ? v[0] - '0' : -1;
}

template <int MODE>
int launch_pair_mode(const CUtensorMap &ma, const CUtensorMap &mb, const GArgs &g, cudaStream_t stream) {
    static bool configured[64] = {false};
    int dev = 0;
    PMOE_CUDA_OK(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        PMOE_CUDA_OK(cudaFuncSetAttribute(moe_bwd_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(PAIR_SMEM_BYTES)));
        configured[dev] = true;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(2);
    int max_clusters = 0;
    PMOE_CUDA_OK(cudaOccupancyMaxActiveClusters(&max_clusters, moe_bwd_pair_kernel<MODE>, &cfg));
    if (max_clusters < 1) return set_error(PMOE_ERR_CUDA, "no CTA pair of the backward GEMM kernel fits on this device");
    // upper bound of the tile count known on the host (the row-space modes read theirs on the device)
    const long long tiles = is_wgrad(g.mode) ? static_cast<long long>(g.E) * ((g.c_rows + 255) / 256) * g.n_tiles
                                                 : static_cast<long long>(g.sorted_num / 256 + 1) * g.n_tiles;
    cfg.gridDim = dim3(2 * static_cast<unsigned>(std::min<long long>(tiles, max_clusters)));
    PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, moe_bwd_pair_kernel<MODE>, ma, mb, g));
    return PMOE_OK;
}

int launch_pair(const CUtensorMap &ma, const CUtensorMap &mb, const GArgs &g, cudaStream_t stream) {
    switch (g.mode) {
        case MODE_NT_STORE: return launch_pair_mode<MODE_NT_STORE>(ma, mb, g, stream);
        case MODE_NN_SWIGLU: return launch_pair_mode<MODE_NN_SWIGLU>(ma, mb, g, stream);
        case MODE_NN_STORE: return launch_pair_mode<MODE_NN_STORE>(ma, mb, g, stream);
        case MODE_WGRAD: return launch_pair_mode<MODE_WGRAD>(ma, mb, g, stream);
        default: return launch_pair_mode<MODE_WGRAD_X>(ma, mb, g, stream);
    }
}

int bf16_map(CUtensorMap *m, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows, const char *what) {
    return make_tmap_2d(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, rows, cols, box_rows, 64,
                        CU_TENSOR_MAP_SWIZZLE_128B, what);
}

}  // namespace

// which steps of the backward pass run (pmoe_debug_set_backward_mask): 1 row maps + gathers, 2 gate/up recompute,
// 4 d_act + SwiGLU derivative, 8 d_w2, 16 d_xs, 32 d_w1, 64 d_x combine
int g_bwd_mask = 127;

int wait_ns_store_bwd(unsigned long long ns) {
    PMOE_CUDA_OK(cudaMemcpyToSymbol(g_wait_ns, &ns, sizeof(ns)));
    return PMOE_OK;
}

int status_fetch_bwd(int *value, bool reset) {
    if (value) PMOE_CUDA_OK(cudaMemcpyFromSymbol(value, g_status_bwd, sizeof(int)));
    if (reset) {
        const int zero = 0;
        PMOE_CUDA_OK(cudaMemcpyToSymbol(g_status_bwd, &zero, sizeof(int)));
    }
    return PMOE_OK;
}

}  // namespace pmoe

extern "C" int pmoe_debug_set_backward_mask(int mask) {
    const int old = pmoe::g_bwd_mask;
    pmoe::g_bwd_mask = mask & 127;
    return old;
}

extern "C" size_t pmoe_fused_moe_bf16_backward_workspace_bytes(int T, int K, int N, int num_experts, int top_k,
                                                               int sorted_num) {
    if (T <= 0 || K <= 0 || N <= 0 || num_experts <= 0 || top_k <= 0 || sorted_num <= 0) return 0;
    return pmoe::plan_backward(T, K, N, num_experts, top_k, sorted_num).total;
}

extern "C" int pmoe_fused_moe_bf16_backward_ex(const void *x, const void *w1, const void *w2, const void *d_out,
                                               const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                               const int32_t *num_tokens_post_padded, const float *topk_weights,
                                               int top_k, int T, int K, int N, int num_experts, int sorted_num,
                                               void *d_x, void *d_w1, void *d_w2, float *d_topk_weights,
                                               const void *gate_up, int dw_dtype, int accumulate_dw, void *workspace,
                                               size_t workspace_bytes, pmoe_stream_t stream_) {
    using namespace pmoe;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PMOE_REQUIRE(dw_dtype == PMOE_DTYPE_BF16 || dw_dtype == PMOE_DTYPE_F32, PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16_backward: dw_dtype must be PMOE_DTYPE_BF16 or PMOE_DTYPE_F32");
    const bool dw_f32 = dw_dtype == PMOE_DTYPE_F32, dw_extended = dw_f32 || accumulate_dw != 0;
    PMOE_REQUIRE(x && w1 && w2 && d_out && sorted_token_ids && expert_ids && num_tokens_post_padded && topk_weights &&
                     d_x && d_w1 && d_w2,
                 PMOE_ERR_BAD_ARG, "fused_moe_bf16_backward: null pointer");
    PMOE_REQUIRE(T >= 0 && K > 0 && N > 0 && num_experts > 0 && top_k > 0 && sorted_num >= 0, PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16_backward: negative or zero size");
    PMOE_REQUIRE(num_experts <= 1024, PMOE_ERR_UNSUPPORTED,
                 "fused_moe_bf16_backward: at most 1024 experts (as moe_align), got %d", num_experts);
    PMOE_REQUIRE(K % 64 == 0 && N % 128 == 0, PMOE_ERR_UNSUPPORTED,
                 "fused_moe_bf16_backward: K must be a multiple of 64 and N of 128, got K=%d N=%d", K, N);
    PMOE_REQUIRE(sorted_num % 128 == 0, PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16_backward: sorted_num must be a multiple of block_m = 128, got %d", sorted_num);
    const uintptr_t all = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w1) |
                          reinterpret_cast<uintptr_t>(w2) | reinterpret_cast<uintptr_t>(d_out) |
                          reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_w1) |
                          reinterpret_cast<uintptr_t>(d_w2);
    PMOE_REQUIRE((all & 15) == 0, PMOE_ERR_BAD_ARG, "fused_moe_bf16_backward: tensors must be 16-byte aligned");
    PMOE_REQUIRE(((reinterpret_cast<uintptr_t>(d_w1) | reinterpret_cast<uintptr_t>(d_w2)) & 31) == 0, PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16_backward: d_w1 and d_w2 must be 32-byte aligned (256-bit stores)");
    const int H = N / 2, E = num_experts;
    const size_t w_elem = dw_f32 ? 4 : 2;
    const size_t w1_bytes = static_cast<size_t>(E) * N * K * w_elem, w2_bytes = static_cast<size_t>(E) * K * H * w_elem;
    if (T == 0 || sorted_num == 0) {   // no routed row: every gradient is zero
        if (!accumulate_dw) {
            PMOE_CUDA_OK(cudaMemsetAsync(d_w1, 0, w1_bytes, stream));
            PMOE_CUDA_OK(cudaMemsetAsync(d_w2, 0, w2_bytes, stream));
        }
        return PMOE_OK;
    }
    const BwdLayout lay = plan_backward(T, K, N, E, top_k, sorted_num);
    PMOE_REQUIRE(workspace && workspace_bytes >= lay.total, PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16_backward: workspace of %zu bytes required, got %zu", lay.total, workspace_bytes);
    PMOE_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 1023) == 0, PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16_backward: workspace must be 1024-byte aligned");
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    auto *xs = reinterpret_cast<__nv_bfloat16 *>(ws + lay.xs);
    auto *dos = reinterpret_cast<__nv_bfloat16 *>(ws + lay.dos);
    // the pre-activations kept by the forward call (pmoe_fused_moe_bf16_keep_ws), or recomputed into the workspace
    PMOE_REQUIRE((reinterpret_cast<uintptr_t>(gate_up) & 31) == 0, PMOE_ERR_BAD_ARG,
                 "fused_moe_bf16_backward: gate_up must be 32-byte aligned");
    auto *gu = gate_up ? const_cast<__nv_bfloat16 *>(static_cast<const __nv_bfloat16 *>(gate_up))
                       : reinterpret_cast<__nv_bfloat16 *>(ws + lay.gu);
    auto *dgu = reinterpret_cast<__nv_bfloat16 *>(ws + lay.dgu);
    auto *actw = reinterpret_cast<__nv_bfloat16 *>(ws + lay.actw);
    auto *inv = reinterpret_cast<int32_t *>(ws + lay.inv);
    auto *eblk = reinterpret_cast<int32_t *>(ws + lay.eblk);
    auto *pair_list = reinterpret_cast<int32_t *>(ws + lay.pair_list);
    auto *single_list = reinterpret_cast<int32_t *>(ws + lay.single_list);
    auto *counts = reinterpret_cast<int32_t *>(ws + lay.counts);
    auto *live_list = reinterpret_cast<int32_t *>(ws + lay.live_list);
    const uint64_t R = static_cast<uint64_t>(sorted_num);

    const int mask = g_bwd_mask;
    const int pm = pairs_mode();
    const bool pairs = pm >= 0 ? pm >= 1 : static_cast<long long>(T) * top_k >= 256ll * E;   // weight gradients
    const bool row_pairs = pm == 2;
    const int copy_grid = 8 * sm_count();
    if (mask & 1) {
        PMOE_CUDA_OK(cudaMemsetAsync(inv, 0xFF, static_cast<size_t>(T) * top_k * sizeof(int32_t), stream));
        PMOE_CUDA_OK(cudaMemsetAsync(eblk, 0, 2 * static_cast<size_t>(E) * sizeof(int32_t), stream));
        const int small_grid = std::max(1, std::min(sorted_num / 256 + 1, 8 * sm_count()));
        row_maps_kernel<<<small_grid, 256, 0, stream>>>(sorted_token_ids, expert_ids, num_tokens_post_padded,
                                                        sorted_num, top_k, T, E, inv, eblk);
        PMOE_CUDA_OK(cudaGetLastError());
        live_items_kernel<<<1, 1024, 0, stream>>>(eblk, E, live_list, counts + 2);
        PMOE_CUDA_OK(cudaGetLastError());
        if (row_pairs) {
            pair_items_kernel<<<1, 1024, 0, stream>>>(eblk, E, pair_list, single_list, counts);
            PMOE_CUDA_OK(cudaGetLastError());
        }
        const bool wide = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(d_out)) & 31) == 0;
        (wide ? gather_token_rows_kernel<true> : gather_token_rows_kernel<false>)<<<copy_grid, 256, 0, stream>>>(
            static_cast<const __nv_bfloat16 *>(x), static_cast<const __nv_bfloat16 *>(d_out), sorted_token_ids,
            num_tokens_post_padded, sorted_num, top_k, T, K, xs, dos);
        PMOE_CUDA_OK(cudaGetLastError());
    }
    if ((mask & 4) && d_topk_weights)
        PMOE_CUDA_OK(cudaMemsetAsync(d_topk_weights, 0, static_cast<size_t>(T) * top_k * sizeof(float), stream));

    CUtensorMap xs_k, xs_mn, dos_k, dos_mn, dgu_k, dgu_mn, actw_mn, w1_k, w1_mn, w2_mn, w1_k128;
    if (int rc = bf16_map(&xs_k, xs, R, K, 128, "xs rows")) return rc;
    if (int rc = bf16_map(&xs_mn, xs, R, K, 64, "xs boxes")) return rc;
    if (int rc = bf16_map(&dos_k, dos, R, K, 128, "d_out rows")) return rc;
    if (int rc = bf16_map(&dos_mn, dos, R, K, 64, "d_out boxes")) return rc;
    if (int rc = bf16_map(&dgu_k, dgu, R, N, 128, "d_gu rows")) return rc;
    if (int rc = bf16_map(&dgu_mn, dgu, R, N, 64, "d_gu boxes")) return rc;
    if (int rc = bf16_map(&actw_mn, actw, R, H, 64, "act boxes")) return rc;
    if (int rc = bf16_map(&w1_k, w1, static_cast<uint64_t>(E) * N, K, 256, "w1 rows")) return rc;
    if (int rc = bf16_map(&w1_mn, w1, static_cast<uint64_t>(E) * N, K, 64, "w1 boxes")) return rc;
    if (int rc = bf16_map(&w2_mn, w2, static_cast<uint64_t>(E) * K, H, 64, "w2 boxes")) return rc;
    if (int rc = bf16_map(&w1_k128, w1, static_cast<uint64_t>(E) * N, K, 128, "w1 half tiles")) return rc;

    GArgs base{};
    base.sorted_ids = sorted_token_ids, base.expert_ids = expert_ids, base.npp = num_tokens_post_padded;
    base.sorted_num = sorted_num, base.eblk = eblk, base.topk_weights = topk_weights;
    base.top_k = top_k, base.tokens = T, base.E = E, base.H = H, base.N = N;
    // A row-space GEMM on CTA pairs is two launches: the pairs of row blocks, then the odd last blocks of the experts
    // on the one-CTA kernel (tcgen05 does not allow cta_group::1 and ::2 in one kernel)
    auto launch_rows = [&](const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mb_pair, GArgs g) -> int {
        if (!row_pairs) {
            g.items = live_list, g.item_count = counts + 2;
            return launch_gemm(ma, mb, g, stream);
        }
        g.items = pair_list, g.item_count = counts;
        if (int rc = launch_pair(ma, mb_pair, g, stream)) return rc;
        g.items = single_list, g.item_count = counts + 1;
        return launch_gemm(ma, mb, g, stream);
    };

    if ((mask & 2) && !gate_up) {   // gate | up pre-activations: gu = xs . W1[e]^T
        GArgs g = base;
        g.mode = MODE_NT_STORE, g.ksteps = K / 64, g.n_tiles = (N + 255) / 256, g.b_rows_per_expert = N;
        g.c = gu, g.ldc = N, g.c_cols = N;
        if (int rc = launch_rows(xs_k, w1_k, w1_k128, g)) return rc;
    }
    if (mask & 4) {   // d_act = wt * (dos . W2[e]) -> d_gu, wt * act, d_wt
        GArgs g = base;
        g.mode = MODE_NN_SWIGLU, g.ksteps = K / 64, g.n_tiles = (H + 255) / 256, g.b_rows_per_expert = K;
        g.gu = gu, g.dgu = dgu, g.actw = actw, g.dwt = d_topk_weights;
        if (int rc = launch_rows(dos_k, w2_mn, w2_mn, g)) return rc;
    }
    if (mask & 8) {   // d_W2[e] [K, H] = dos_e^T . (wt * act)_e
        GArgs g = base;
        g.mode = dw_extended ? MODE_WGRAD_X : MODE_WGRAD, g.m_tiles = (K + 127) / 128, g.n_tiles = (H + 255) / 256;
        g.c = static_cast<__nv_bfloat16 *>(d_w2), g.ldc = H, g.c_cols = H, g.c_rows = K;
        g.c_f32 = dw_f32 ? static_cast<float *>(d_w2) : nullptr, g.accumulate = accumulate_dw ? 1 : 0;
        if (int rc = (pairs ? launch_pair : launch_gemm)(dos_mn, actw_mn, g, stream)) return rc;
    }
    if (mask & 16) {   // d_xs = d_gu . W1[e], written over dos (dead from here on)
        GArgs g = base;
        g.mode = MODE_NN_STORE, g.ksteps = N / 64, g.n_tiles = (K + 255) / 256, g.b_rows_per_expert = N;
        g.c = dos, g.ldc = K, g.c_cols = K;
        if (int rc = launch_rows(dgu_k, w1_mn, w1_mn, g)) return rc;
    }
    if (mask & 32) {   // d_W1[e] [N, K] = d_gu_e^T . xs_e
        GArgs g = base;
        g.mode = dw_extended ? MODE_WGRAD_X : MODE_WGRAD, g.m_tiles = (N + 127) / 128, g.n_tiles = (K + 255) / 256;
        g.c = static_cast<__nv_bfloat16 *>(d_w1), g.ldc = K, g.c_cols = K, g.c_rows = N;
        g.c_f32 = dw_f32 ? static_cast<float *>(d_w1) : nullptr, g.accumulate = accumulate_dw ? 1 : 0;
        if (int rc = (pairs ? launch_pair : launch_gemm)(dgu_mn, xs_mn, g, stream)) return rc;
    }
    if (mask & 64) {
        combine_dx_kernel<<<copy_grid, 256, 0, stream>>>(dos, inv, top_k, T, K, static_cast<__nv_bfloat16 *>(d_x));
        PMOE_CUDA_OK(cudaGetLastError());
    }
    return PMOE_OK;
}

extern "C" int pmoe_fused_moe_bf16_backward(const void *x, const void *w1, const void *w2, const void *d_out,
                                            const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                            const int32_t *num_tokens_post_padded, const float *topk_weights,
                                            int top_k, int T, int K, int N, int num_experts, int sorted_num,
                                            void *d_x, void *d_w1, void *d_w2, float *d_topk_weights,
                                            const void *gate_up, void *workspace, size_t workspace_bytes,
                                            pmoe_stream_t stream) {
    return pmoe_fused_moe_bf16_backward_ex(x, w1, w2, d_out, sorted_token_ids, expert_ids, num_tokens_post_padded,
                                           topk_weights, top_k, T, K, N, num_experts, sorted_num, d_x, d_w1, d_w2,
                                           d_topk_weights, gate_up, PMOE_DTYPE_BF16, 0, workspace, workspace_bytes, stream);
}
