// mxfp8 (OCP-MX: e4m3 values, one e8m0 scale per 32 K-elements) fused MoE FFN for sm_100a.
//
// Replaces the kernels and launcher of prime_moe/csrc/kernels/fused_moe_mxfp8_kernel.cu
// (gather_x_mxfp8_kernel :56-80, fused_moe_mxfp8_kernel :82-503, fused_moe_mxfp8_down_kernel :513-679,
// launch_fused_moe_mxfp8_kernel :681-866) behind pmoe_fused_moe_mxfp8.
//
// Same decomposition and warp roles as the bf16 kernels (moe_bf16.cu): persistent CTAs, warp 0 = TMA
// producer, warp 1 = tcgen05.mma issuer, 8 epilogue warps. Differences:
//   * MMA = tcgen05.mma.kind::mxf8f6f4.block_scale, M128 x N256 x K32; a ring slot holds 128 K-bytes:
//     A 128x128 B + B 256x128 B (128-byte swizzle) + three 512-byte scale tiles (A, B gate half / first
//     128 rows, B up half / last 128 rows).
//   * scale tiles travel global -> shared by untiled bulk copies, shared -> TMEM by
//     tcgen05.cp.32x128b.warpx4 (4 TMEM columns per tile), issued by the MMA thread ahead of the four
//     MMAs of the slot; the instruction descriptor's scale-factor ids select the K-block byte.
//     Eight rotating 16-column TMEM regions keep the scales of in-flight slots apart.
//   * TMEM: one 256-column accumulator (the scale regions leave no room for a second one). The
//     epilogue warps first DRAIN the accumulator into registers (128 fp32 per thread), hand it back to
//     the MMA thread, and only then do their arithmetic and stores, so the next tile's main loop
//     overlaps all of the epilogue except the drain itself.
//   * gate/up epilogue: SwiGLU in fp32, then per row and per 32 columns the MX re-quantisation of the
//     reference (fused_moe_mxfp8_kernel.cu:4-20, 375-403): e = clamp(exponent(amax) - 8, 0, 254),
//     q = satfinite_e4m3(v * 2^(127-e)); e4m3 tile -> TMA store, scale bytes -> 512-byte tiles.
//   * routing weight stays fp32 (as in the reference's mxfp8 path).
//
// Scale tile layout everywhere (prime_moe/__init__.py:106-115): 128 rows x 4 K-blocks, byte
// (r%32)*16 + (r/32)*4 + kb.
#include <cuda_fp8.h>
#include <stdio.h>

#include <algorithm>

#include "host_common.h"
#include "ptx.cuh"
#include "tile_sched.cuh"

namespace pmoe {

__device__ int g_status_mxfp8 = 0;

namespace {

constexpr int BM = kBlockM;
constexpr int BKB = 128;                         // K bytes (= e4m3 elements) per ring slot
constexpr uint32_t A_BYTES = BM * BKB;           // 16 KB
constexpr uint32_t B_BYTES = 256 * BKB;          // 32 KB
constexpr uint32_t SF_TILE = 512;
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES + 2048;   // 50 KB: + SFA, SFB(2), pad
constexpr uint32_t STAGE_TX_BYTES = A_BYTES + B_BYTES + 3 * SF_TILE;
constexpr uint32_t ACT_TILE_BYTES = 128 * 128;   // e4m3 activation tile (store staging / fused A operand)
constexpr int MAX_STAGES = 4;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t SF_TMEM_BASE = 256;           // columns [256, 384): eight 16-column scale regions
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + EPI_WARPS * 32;
constexpr int GATHER_THREADS = 128;             // optional LSU gather warps of the gate/up kernel
constexpr int UP_MAX_THREADS = THREADS + GATHER_THREADS;
constexpr uint32_t BAR_BYTES = 256;
constexpr uint32_t RED_ROW_BYTES = 256 + 16;              // down epilogue staging: 128 bf16 per thread, padded
constexpr uint32_t RED_STAGE_BYTES = EPI_WARPS * 32 * RED_ROW_BYTES;

struct Args {
    const int32_t *sorted_ids;
    const int32_t *expert_ids;
    const int32_t *npp;
    const float *topk_weights;
    __nv_bfloat16 *out;
    float *acc32;
    const uint8_t *w_scales;    // blocked, [E*N/128][K/128][512]
    const uint8_t *w2_scales;   // blocked, [E*K/128][H/128][512]
    const uint8_t *xsf_tiles;   // up kernel (split): [blocks][K/128][512] re-tiled activation scales
    uint8_t *act_sf;            // [blocks][H/128][512] scales of the re-quantised activation
    int M, K, N, H;
    int top_k;
    int sorted_num;
    int stages;
    int zero_out;
    int use_pdl;
    int bulk_reduce;   // down kernel: reduce into `out` with cp.reduce.async.bulk from a staging tile
    const int32_t *live_rows;   // optional: rows of `out` in use (only those are zeroed)
    const uint8_t *x;           // gate/up kernel with the in-kernel row gather: e4m3 activations [M, K] ...
    const uint8_t *x_scales;    // ... and their row-major e8m0 scales [M, K/32]
    int lsu_gather;             // gate/up kernel: A rows and A scale tiles gathered from x by four extra warps
    int short_boxes;   // split kernels: row blocks with <= SHORT_ROWS routed rows move only those rows of the A
                       // operand and of the activation tile (the rest of a 128-row block is padding)
};

constexpr int SHORT_ROWS = 32;
constexpr uint32_t SHORT_A_BYTES = SHORT_ROWS * BKB;

// routed rows come first in a block, so the block is short when row SHORT_ROWS is already padding
__device__ __forceinline__ bool block_is_short(const Args &a, int blk, int what = 1) {
    return (a.short_boxes & what) && a.sorted_ids[blk * BM + SHORT_ROWS] < 0;
}

struct Smem {
    uint32_t ring, act, bars;
    __device__ __forceinline__ uint32_t a(int s) const { return ring + s * STAGE_BYTES; }
    __device__ __forceinline__ uint32_t b(int s) const { return ring + s * STAGE_BYTES + A_BYTES; }
    __device__ __forceinline__ uint32_t sfa(int s) const { return ring + s * STAGE_BYTES + A_BYTES + B_BYTES; }
    __device__ __forceinline__ uint32_t sfb(int s) const { return sfa(s) + SF_TILE; }
    __device__ __forceinline__ uint32_t full(int s) const { return bars + 8 * s; }
    __device__ __forceinline__ uint32_t empty(int s) const { return bars + 8 * (MAX_STAGES + s); }
    __device__ __forceinline__ uint32_t misc(int i) const { return bars + 8 * (2 * MAX_STAGES + i); }
    __device__ __forceinline__ uint32_t tmem_slot() const { return bars + 8 * (2 * MAX_STAGES + 12); }
};
constexpr uint32_t ACT_EXTRA = ACT_TILE_BYTES + 1024;   // activation tile + one 512-byte scale tile (fused), padded
__device__ __forceinline__ Smem carve(const uint8_t *raw, int stages, uint32_t extra) {
    Smem s;
    s.ring = (smem_u32(raw) + 1023u) & ~1023u;
    s.act = s.ring + stages * STAGE_BYTES;
    s.bars = s.act + extra;   // extra = ACT_EXTRA (up / fused), reduction staging (down) or 0
    return s;
}
size_t smem_bytes(int stages, uint32_t extra) {
    return 1024 + static_cast<size_t>(stages) * STAGE_BYTES + extra + BAR_BYTES;
}

__device__ __forceinline__ void drain_fills(const Smem &sm, int stages, long long issued) {
    const long long first = issued > stages ? issued - stages : 0;
    for (long long f = first; f < issued; ++f) {
        const uint32_t bar = sm.full(static_cast<int>(f % stages));
        const uint32_t parity = static_cast<uint32_t>((f / stages) & 1);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(bar, parity)) {
            if (globaltimer_ns() - t0 > 20000000ull) break;
        }
    }
}

__device__ __forceinline__ void ld32(float *dst, uint32_t taddr) {
    tmem_ld_32x32(*reinterpret_cast<float(*)[32]>(dst), taddr);
}

// epilogue warps poll and arrive through lane 0 only: 8 pollers / arrivals per barrier instead of 256
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, int *status, int code, int lane) {
    bool ok = true;
    if (lane == 0) ok = mbar_wait(bar, parity, status, code);
    return __shfl_sync(0xffffffffu, ok, 0);
}
__device__ __forceinline__ void warp_arrive(uint32_t bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void warp_arrive_cluster(uint32_t cluster_bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(cluster_bar);
}

// MX block scale of 32 values: returns the biased e8m0 exponent, *inv = 2^(127 - e)
__device__ __forceinline__ uint32_t mx_block_scale(float amax, float *inv) {
    int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu) - 8;
    e = max(0, min(e, 254));
    const uint32_t field = static_cast<uint32_t>(254 - e);
    *inv = __uint_as_float(field ? field << 23 : 0x00400000u);   // 2^-127 is subnormal
    return static_cast<uint32_t>(e);
}
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

// one ring slot -> TMEM scale region, then four K32 MMAs
__device__ __forceinline__ void issue_slot(uint32_t d, uint32_t a_smem, uint32_t b_smem, uint32_t sfa_smem,
                                           uint32_t sfb0_smem, uint32_t sfb1_smem, uint32_t tmem_base,
                                           long long fill, bool first, uint32_t idesc, int n_sfb_tiles) {
    const uint32_t sfa_t = tmem_base + SF_TMEM_BASE + 16u * static_cast<uint32_t>(fill & 7);
    const uint32_t sfb_t = sfa_t + 4;
    tmem_cp_sf_32x128b_warpx4(sfa_t, smem_desc_sf(sfa_smem));
    tmem_cp_sf_32x128b_warpx4(sfb_t, smem_desc_sf(sfb0_smem));
    if (n_sfb_tiles > 1) tmem_cp_sf_32x128b_warpx4(sfb_t + 4, smem_desc_sf(sfb1_smem));
#pragma unroll
    for (uint32_t kb = 0; kb < 4; ++kb)
        umma_mxf8(d, smem_desc_sw128(a_smem + kb * 32), smem_desc_sw128(b_smem + kb * 32),
                  idesc_with_sf_ids(idesc, kb, kb), sfa_t, sfb_t, (!first || kb != 0) ? 1u : 0u);
}

// ---------------------------------------------------------------------------------------------
// pre-pass of the split pipeline: x_sorted[row] = x[token(row)] (e4m3 bytes) and the row-major
// activation scales re-tiled into 512-byte tiles [block][K/128]. One warp per row.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gather_rows_mxfp8_kernel(const uint8_t *__restrict__ x, const uint8_t *__restrict__ x_scales,
                         uint8_t *__restrict__ x_sorted, uint8_t *__restrict__ xsf_tiles, const Args a) {
    pdl_launch_dependents();   // the gate/up (or fused) kernel may set itself up; it waits for this grid before loading
    const int warps_per_cta = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rows = live_row_blocks(a.npp, a.sorted_num) * BM;
    const int chunks = a.K / 16;
    const int kblocks = a.K / 32;
    for (int row = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_cta) {
        const int pair = a.sorted_ids[row];
        const int tok = pair >= 0 ? pair / a.top_k : -1;
        // padding rows (values and scales) are not copied: they only feed accumulator rows that are never
        // written out, and every output row depends on its own A row alone
        if (tok < 0 || tok >= a.M) continue;
        const int4 *src = reinterpret_cast<const int4 *>(x + static_cast<size_t>(tok) * a.K);
        int4 *dst = reinterpret_cast<int4 *>(x_sorted + static_cast<size_t>(row) * a.K);
        for (int ch = lane; ch < chunks; ch += 32) dst[ch] = __ldg(src + ch);
        const int r = row & 127;
        uint8_t *tiles = xsf_tiles + static_cast<size_t>(row >> 7) * (a.K / 128) * SF_TILE;
        const uint8_t *srow = x_scales + static_cast<size_t>(tok) * kblocks;
        for (int kb = lane; kb < kblocks; kb += 32)
            tiles[(kb >> 2) * SF_TILE + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = srow[kb];
    }
}

// ---------------------------------------------------------------------------------------------
// up kernel (split): misc barriers 0 tmem_full | 1 tmem_empty | 2 staged | 3 stage_free
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(UP_MAX_THREADS, 1)
moe_up_mxfp8_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w1,
                    const __grid_constant__ CUtensorMap map_act, const __grid_constant__ CUtensorMap map_x_short,
                    const __grid_constant__ CUtensorMap map_act_short, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const Smem sm = carve(smem_raw, a.stages, ACT_EXTRA);
    int *status = &g_status_mxfp8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int epi_threads = EPI_WARPS * 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(sm.full(s), a.lsu_gather ? 1 + GATHER_THREADS : 1);
            mbar_init(sm.empty(s), 1);
        }
        mbar_init(sm.misc(0), 1);
        mbar_init(sm.misc(1), EPI_WARPS);
        mbar_init(sm.misc(2), EPI_WARPS);
        mbar_init(sm.misc(3), 1);
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

    const int m_blocks = live_row_blocks(a.npp, a.sorted_num);
    const int n_tiles = a.H / 128;
    const int num_tiles = m_blocks * n_tiles;
    const int ksteps = a.K / BKB;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            long long issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const Coord c = tile_coord(t, m_blocks, n_tiles);
                const int e = a.expert_ids[c.m_blk];
                const int row_gate = e * a.N + c.n_tile * 128;
                const int row_up = row_gate + a.H;
                const uint8_t *sf_gate = a.w_scales + static_cast<size_t>(row_gate >> 7) * ksteps * SF_TILE;
                const uint8_t *sf_up = a.w_scales + static_cast<size_t>(row_up >> 7) * ksteps * SF_TILE;
                const uint8_t *sf_x = a.xsf_tiles + static_cast<size_t>(c.m_blk) * ksteps * SF_TILE;
                const bool short_a = !a.lsu_gather && block_is_short(a, c.m_blk);
                for (int ks = 0; ks < ksteps; ++ks) {
                    ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                    if (!ok) break;
                    if (a.lsu_gather) {   // the A tile and its scale tile come from the gather warps
                        mbar_arrive_expect_tx(sm.full(s), B_BYTES + 2 * SF_TILE);
                    } else {
                        mbar_arrive_expect_tx(sm.full(s), short_a ? STAGE_TX_BYTES - A_BYTES + SHORT_A_BYTES : STAGE_TX_BYTES);
                        tma_load_2d(sm.a(s), short_a ? &map_x_short : &map_x, sm.full(s), ks * BKB, c.m_blk * BM);
                        bulk_load_1d(sm.sfa(s), sf_x + static_cast<size_t>(ks) * SF_TILE, SF_TILE, sm.full(s));
                    }
                    tma_load_2d(sm.b(s), &map_w1, sm.full(s), ks * BKB, row_gate);
                    tma_load_2d(sm.b(s) + B_BYTES / 2, &map_w1, sm.full(s), ks * BKB, row_up);
                    bulk_load_1d(sm.sfb(s), sf_gate + static_cast<size_t>(ks) * SF_TILE, SF_TILE, sm.full(s));
                    bulk_load_1d(sm.sfb(s) + SF_TILE, sf_up + static_cast<size_t>(ks) * SF_TILE, SF_TILE, sm.full(s));
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
            constexpr uint32_t idesc = idesc_mxf8_f32(128, 256);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            long long fill = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
                ok = mbar_wait(sm.misc(1), (it & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                for (int ks = 0; ks < ksteps; ++ks, ++fill) {
                    ok = mbar_wait(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
                    issue_slot(tmem_base, sm.a(s), sm.b(s), sm.sfa(s), sm.sfb(s), sm.sfb(s) + SF_TILE, tmem_base, fill,
                               ks == 0, idesc, 2);
                    umma_commit(sm.empty(s));
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit(sm.misc(0));
            }
        }
        __syncwarp();
    } else if (warp >= 2 + EPI_WARPS) {
        // ---------------- LSU gather warps: A rows and the A scale tile straight from x / x_scales ----------------
        // As in the bf16 gate/up kernel: 8 consecutive lanes copy the eight 16-byte chunks of one 128-byte row segment
        // (thread g serves rows (g>>3) + 16*i) into the 128-byte-swizzled tile; in addition thread g copies the four
        // scale bytes of row g for this k-step into the 512-byte scale tile (byte (r%32)*16 + (r/32)*4 + kb). cp.async
        // writes through the generic proxy, tcgen05.mma / tcgen05.cp read through the async proxy: each thread waits
        // for its own copies of a slot (lagging behind the slots it is issuing), fences, then arrives on `full`.
        const int g = threadIdx.x - 64 - epi_threads;
        const int q = g >> 3, chunk = g & 7;
        const int lag = min(2, a.stages - 1);
        const int kblocks = a.K / 32;
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
            const Coord c = tile_coord(t, m_blocks, n_tiles);
            const uint8_t *src[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int pair = a.sorted_ids[c.m_blk * BM + q + 16 * i];
                int tok = pair >= 0 ? pair / a.top_k : 0;     // padding rows read token 0; their result is dropped
                if (tok >= a.M) tok = 0;
                src[i] = a.x + static_cast<size_t>(tok) * a.K + chunk * 16;
            }
            const int pair_g = a.sorted_ids[c.m_blk * BM + g];
            int tok_g = pair_g >= 0 ? pair_g / a.top_k : 0;
            if (tok_g >= a.M) tok_g = 0;
            const uint8_t *ssrc = a.x_scales + static_cast<size_t>(tok_g) * kblocks;
            const uint32_t sdst = (g & 31) * 16 + (g >> 5) * 4;
            for (int ks = 0; ks < ksteps; ++ks) {
                ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                if (!ok) break;
                const uint32_t dst = sm.a(s) + q * 128 + ((chunk ^ (q & 7)) << 4);
#pragma unroll
                for (int i = 0; i < 8; ++i) cp_async_16(dst + i * 16 * 128, src[i] + ks * BKB);
                cp_async_4(sm.sfa(s) + sdst, ssrc + ks * 4);
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
        const int ew = warp - 2;
        const int et = threadIdx.x - 64;
        const uint32_t lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;
        const int cg = ew >> 2;          // 0: activation columns [0,64), 1: [64,128)
        if (a.zero_out) {
            int4 *o4 = reinterpret_cast<int4 *>(a.out);
            const long long n4 = static_cast<long long>(a.live_rows ? max(0, min(a.M, *a.live_rows)) : a.M) * a.K / 8;
            const int4 z = make_int4(0, 0, 0, 0);
            for (long long i = static_cast<long long>(blockIdx.x) * epi_threads + et; i < n4;
                 i += static_cast<long long>(gridDim.x) * epi_threads)
                o4[i] = z;
        }
        int it = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            const Coord c = tile_coord(t, m_blocks, n_tiles);
            if (!warp_wait(sm.misc(0), it & 1, status, ST_TIMEOUT_TMEM_FULL, lane)) break;
            tc_fence_after();
            float g[64], u[64];
            ld32(g, tmem_addr(tmem_base, lane_base, cg * 64));
            ld32(g + 32, tmem_addr(tmem_base, lane_base, cg * 64 + 32));
            ld32(u, tmem_addr(tmem_base, lane_base, 128 + cg * 64));
            ld32(u + 32, tmem_addr(tmem_base, lane_base, 128 + cg * 64 + 32));
            tmem_ld_wait();
            tc_fence_before();
            warp_arrive(sm.misc(1), lane);   // accumulator drained: the next tile's main loop may start
#pragma unroll
            for (int i = 0; i < 64; ++i) g[i] = swiglu(g[i], u[i]);
            if (!warp_wait(sm.misc(3), (it & 1) ^ 1, status, ST_TIMEOUT_ACT, lane)) break;   // staging tile free
            uint8_t *sf_tile = a.act_sf + (static_cast<size_t>(c.m_blk) * n_tiles + c.n_tile) * SF_TILE;
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(g[blk * 32 + i]));
                float inv;
                const uint32_t e = mx_block_scale(amax, &inv);
                sf_tile[(row & 31) * 16 + (row >> 5) * 4 + cg * 2 + blk] = static_cast<uint8_t>(e);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float *v = g + blk * 32 + j * 16;
                    const uint32_t chunk16 = static_cast<uint32_t>(cg * 4 + blk * 2 + j);
                    st_shared_v4(sm.act + row * 128 + ((chunk16 ^ (row & 7)) << 4),
                                 pack_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv),
                                 pack_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv),
                                 pack_e4m3x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv),
                                 pack_e4m3x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv));
                }
            }
            fence_proxy_async_smem();
            warp_arrive(sm.misc(2), lane);
            bool stored = true;
            if (et == 0) {
                stored = mbar_wait(sm.misc(2), it & 1, status, ST_TIMEOUT_ACT);
                if (stored) {
                    tma_store_2d(block_is_short(a, c.m_blk, 2) ? &map_act_short : &map_act, sm.act, c.n_tile * 128,
                                 c.m_blk * BM);
                    tma_store_commit();
                    tma_store_wait_read<0>();
                    mbar_arrive(sm.misc(3));
                }
            }
            if (!__shfl_sync(0xffffffffu, stored, 0)) break;   // keep the warp together on the error path
        }
        if (et == 0) tma_store_wait<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// down kernel (split): misc barriers 0 tmem_full | 1 tmem_empty
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS, 1)
moe_down_mxfp8_kernel(const __grid_constant__ CUtensorMap map_act, const __grid_constant__ CUtensorMap map_w2,
                      const __grid_constant__ CUtensorMap map_act_short, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const Smem sm = carve(smem_raw, a.stages, a.bulk_reduce ? RED_STAGE_BYTES : 0u);
    int *status = &g_status_mxfp8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        mbar_init(sm.misc(0), 1);
        mbar_init(sm.misc(1), EPI_WARPS);
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

    if (a.use_pdl) pdl_wait_primary();

    const int m_blocks = live_row_blocks(a.npp, a.sorted_num);
    const int n_tiles = a.K / 256;
    const int num_tiles = m_blocks * n_tiles;
    const int ksteps = a.H / BKB;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            long long issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const Coord c = tile_coord(t, m_blocks, n_tiles);
                const int e = a.expert_ids[c.m_blk];
                const int w2_row = e * a.K + c.n_tile * 256;
                const uint8_t *sf_w0 = a.w2_scales + static_cast<size_t>(w2_row >> 7) * ksteps * SF_TILE;
                const uint8_t *sf_w1 = sf_w0 + static_cast<size_t>(ksteps) * SF_TILE;
                const uint8_t *sf_a = a.act_sf + static_cast<size_t>(c.m_blk) * ksteps * SF_TILE;
                const bool short_a = block_is_short(a, c.m_blk);
                for (int ks = 0; ks < ksteps; ++ks) {
                    ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_arrive_expect_tx(sm.full(s), short_a ? STAGE_TX_BYTES - A_BYTES + SHORT_A_BYTES : STAGE_TX_BYTES);
                    tma_load_2d(sm.a(s), short_a ? &map_act_short : &map_act, sm.full(s), ks * BKB, c.m_blk * BM);
                    tma_load_2d(sm.b(s), &map_w2, sm.full(s), ks * BKB, w2_row);
                    bulk_load_1d(sm.sfa(s), sf_a + static_cast<size_t>(ks) * SF_TILE, SF_TILE, sm.full(s));
                    bulk_load_1d(sm.sfb(s), sf_w0 + static_cast<size_t>(ks) * SF_TILE, SF_TILE, sm.full(s));
                    bulk_load_1d(sm.sfb(s) + SF_TILE, sf_w1 + static_cast<size_t>(ks) * SF_TILE, SF_TILE, sm.full(s));
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
            constexpr uint32_t idesc = idesc_mxf8_f32(128, 256);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            long long fill = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
                ok = mbar_wait(sm.misc(1), (it & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                for (int ks = 0; ks < ksteps; ++ks, ++fill) {
                    ok = mbar_wait(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
                    issue_slot(tmem_base, sm.a(s), sm.b(s), sm.sfa(s), sm.sfb(s), sm.sfb(s) + SF_TILE, tmem_base, fill,
                               ks == 0, idesc, 2);
                    umma_commit(sm.empty(s));
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit(sm.misc(0));
            }
        }
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const uint32_t lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;
        const int cg = ew >> 2;          // output columns [cg*128, cg*128+128) of the 256-wide tile
        int it = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            const Coord c = tile_coord(t, m_blocks, n_tiles);
            const int pair = a.sorted_ids[c.m_blk * BM + row];
            const int tok = pair >= 0 ? pair / a.top_k : 0;
            const bool valid = pair >= 0 && tok < a.M;
            const float wgt = valid ? a.topk_weights[pair] : 0.f;
            __nv_bfloat16 *dst = a.out + static_cast<size_t>(valid ? tok : 0) * a.K + c.n_tile * 256 + cg * 128;
            if (!warp_wait(sm.misc(0), it & 1, status, ST_TIMEOUT_TMEM_FULL, lane)) break;
            tc_fence_after();
            float v[128];
#pragma unroll
            for (int q = 0; q < 4; ++q) ld32(v + q * 32, tmem_addr(tmem_base, lane_base, cg * 128 + q * 32));
            tmem_ld_wait();
            tc_fence_before();
            warp_arrive(sm.misc(1), lane);
            if (a.bulk_reduce) {
                // scaled bf16 row segment -> this thread's padded staging row -> one 256-byte bulk reduction
                const uint32_t red_row = sm.act + (threadIdx.x - 64) * RED_ROW_BYTES;
                tma_store_wait_read<0>();
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    st_shared_v4(red_row + j * 16, pack_bf16x2(wgt * v[j * 8 + 0], wgt * v[j * 8 + 1]),
                                 pack_bf16x2(wgt * v[j * 8 + 2], wgt * v[j * 8 + 3]),
                                 pack_bf16x2(wgt * v[j * 8 + 4], wgt * v[j * 8 + 5]),
                                 pack_bf16x2(wgt * v[j * 8 + 6], wgt * v[j * 8 + 7]));
                fence_proxy_async_smem();
                if (valid) bulk_reduce_add_bf16(dst, red_row, 256);
                tma_store_commit();
                continue;
            }
            if (valid) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    red_add_bf16x8(dst + j * 8, pack_bf16x2(wgt * v[j * 8 + 0], wgt * v[j * 8 + 1]),
                                   pack_bf16x2(wgt * v[j * 8 + 2], wgt * v[j * 8 + 3]),
                                   pack_bf16x2(wgt * v[j * 8 + 4], wgt * v[j * 8 + 5]),
                                   pack_bf16x2(wgt * v[j * 8 + 6], wgt * v[j * 8 + 7]));
            }
        }
        if (a.bulk_reduce) tma_store_wait<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// CTA-pair kernels (bpc == 2; no counterpart in the reference, whose mxfp8 path is bpc=1 only): cluster of
// two CTAs, tcgen05.mma.cta_group::2 with M = 256. A pair owns two consecutive 128-row blocks of one expert
// (moe_align pads experts to 256 rows when bpc == 2) x one 256-column tile. Per k-step each CTA loads ITS
// 128 A rows, ITS half of the B tile (gate/up kernel: even CTA the gate rows, odd CTA the up rows; down
// kernel: 128 of the 256 w2 rows each), its own A scale tile and BOTH B scale tiles (every CTA's tensor
// memory needs the scales of all 256 B rows): 33.5 KB instead of 49.5 KB, which buys a ring of six slots.
// All loads are plain TMA tile loads (.cta_group::2 only routes their completion bytes to the even CTA's
// `full` barrier; the 512-byte scale tiles travel as 1 x 128 boxes of 32-bit words) - no multicast. The even
// CTA issues the scale copies and MMAs for both; slots and the accumulator are handed back to both CTAs by
// multicast tcgen05.commit; both CTAs' epilogues arrive on the even CTA's tmem_empty.
//   misc barriers: 0 tmem_full (each CTA) | 1 tmem_empty (even CTA) | 2 staged | 3 stage_free (up only)
// ---------------------------------------------------------------------------------------------
constexpr uint32_t PAIR_STAGE_BYTES = A_BYTES + B_BYTES / 2 + 2048;          // 34 KB: + SFA, SFB(2), pad
constexpr uint32_t PAIR_TX_BYTES = A_BYTES + B_BYTES / 2 + 3 * SF_TILE;      // bytes one CTA loads per slot
constexpr int PAIR_MAX_STAGES = 6;
constexpr int ST_BAD_PAIR = 8;                                               // the two blocks of a pair differ in expert

struct SmemPair {
    uint32_t ring, act, bars;
    __device__ __forceinline__ uint32_t a(int s) const { return ring + s * PAIR_STAGE_BYTES; }
    __device__ __forceinline__ uint32_t b(int s) const { return ring + s * PAIR_STAGE_BYTES + A_BYTES; }
    __device__ __forceinline__ uint32_t sfa(int s) const { return ring + s * PAIR_STAGE_BYTES + A_BYTES + B_BYTES / 2; }
    __device__ __forceinline__ uint32_t sfb(int s) const { return sfa(s) + SF_TILE; }
    __device__ __forceinline__ uint32_t full(int s) const { return bars + 8 * s; }
    __device__ __forceinline__ uint32_t empty(int s) const { return bars + 8 * (PAIR_MAX_STAGES + s); }
    __device__ __forceinline__ uint32_t misc(int i) const { return bars + 8 * (2 * PAIR_MAX_STAGES + i); }
    __device__ __forceinline__ uint32_t tmem_slot() const { return bars + 8 * (2 * PAIR_MAX_STAGES + 8); }
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

template <bool kUp>
__global__ void __launch_bounds__(THREADS, 1)
moe_pair_mxfp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                      const __grid_constant__ CUtensorMap map_act, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const SmemPair sm = carve_pair(smem_raw, a.stages, kUp ? ACT_EXTRA : (a.bulk_reduce ? RED_STAGE_BYTES : 0u));
    int *status = &g_status_mxfp8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int epi_threads = EPI_WARPS * 32;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        mbar_init(sm.misc(0), 1);
        mbar_init(sm.misc(1), 2 * EPI_WARPS);
        mbar_init(sm.misc(2), EPI_WARPS);
        mbar_init(sm.misc(3), 1);
        fence_mbar_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
        tma_prefetch_desc(&map_sfa);
        tma_prefetch_desc(&map_sfb);
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

    const int m_pairs = live_row_blocks(a.npp, a.sorted_num) / 2;
    const int n_tiles = kUp ? a.H / 128 : a.K / 256;
    const int num_tiles = m_pairs * n_tiles;
    const int ksteps = (kUp ? a.K : a.H) / BKB;
    const int first = blockIdx.x >> 1, step = gridDim.x >> 1;   // this pair's tile sequence

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = first; t < num_tiles && ok; t += step) {
                const Coord c = tile_coord(t, m_pairs, n_tiles);
                const int blk = 2 * c.m_blk + static_cast<int>(rank);
                const int e = a.expert_ids[2 * c.m_blk];
                if (leader && a.expert_ids[2 * c.m_blk + 1] != e) atomicCAS(status, 0, ST_BAD_PAIR);
                int b_row, sfb0, sfb1;   // B rows of this CTA; scale-tile rows of the two 128-row halves of B
                if (kUp) {
                    const int row_gate = e * a.N + c.n_tile * 128;
                    b_row = row_gate + (leader ? 0 : a.H);
                    sfb0 = (row_gate >> 7) * ksteps;
                    sfb1 = ((row_gate + a.H) >> 7) * ksteps;
                } else {
                    const int w2_row = e * a.K + c.n_tile * 256;
                    b_row = w2_row + static_cast<int>(rank) * 128;
                    sfb0 = (w2_row >> 7) * ksteps;
                    sfb1 = sfb0 + ksteps;
                }
                const int sfa0 = blk * ksteps;
                for (int ks = 0; ks < ksteps; ++ks) {
                    ok = mbar_wait_cluster(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                    if (!ok) break;
                    const uint32_t full_leader = mapa_shared(sm.full(s), 0);
                    if (leader) mbar_arrive_expect_tx(sm.full(s), 2 * PAIR_TX_BYTES);
                    tma_load_2d_pair(sm.a(s), &map_a, full_leader, ks * BKB, blk * BM);
                    tma_load_2d_pair(sm.b(s), &map_b, full_leader, ks * BKB, b_row);
                    tma_load_2d_pair(sm.sfa(s), &map_sfa, full_leader, 0, sfa0 + ks);
                    tma_load_2d_pair(sm.sfb(s), &map_sfb, full_leader, 0, sfb0 + ks);
                    tma_load_2d_pair(sm.sfb(s) + SF_TILE, &map_sfb, full_leader, 0, sfb1 + ks);
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
            constexpr uint32_t idesc = idesc_mxf8_f32(256, 256);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            long long fill = 0;
            bool ok = true;
            for (int t = first; t < num_tiles && ok; t += step, ++it) {
                ok = mbar_wait_cluster(sm.misc(1), (it & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                for (int ks = 0; ks < ksteps; ++ks, ++fill) {
                    ok = mbar_wait_cluster(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sfa_t = tmem_base + SF_TMEM_BASE + 16u * static_cast<uint32_t>(fill & 7);
                    const uint32_t sfb_t = sfa_t + 4;
                    tmem_cp_sf_32x128b_warpx4_pair(sfa_t, smem_desc_sf(sm.sfa(s)));
                    tmem_cp_sf_32x128b_warpx4_pair(sfb_t, smem_desc_sf(sm.sfb(s)));
                    tmem_cp_sf_32x128b_warpx4_pair(sfb_t + 4, smem_desc_sf(sm.sfb(s) + SF_TILE));
#pragma unroll
                    for (uint32_t kb = 0; kb < 4; ++kb)
                        umma_mxf8_pair(tmem_base, smem_desc_sw128(sm.a(s) + kb * 32), smem_desc_sw128(sm.b(s) + kb * 32),
                                       idesc_with_sf_ids(idesc, kb, kb), sfa_t, sfb_t, (ks | kb) != 0 ? 1u : 0u);
                    umma_commit_pair(sm.empty(s), 3);
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit_pair(sm.misc(0), 3);
            }
        }
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const int et = threadIdx.x - 64;
        const uint32_t lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;
        const int cg = ew >> 2;
        const uint32_t empty_leader = mapa_shared(sm.misc(1), 0);
        if (kUp && a.zero_out) {
            int4 *o4 = reinterpret_cast<int4 *>(a.out);
            const long long n4 = static_cast<long long>(a.live_rows ? max(0, min(a.M, *a.live_rows)) : a.M) * a.K / 8;
            const int4 z = make_int4(0, 0, 0, 0);
            for (long long i = static_cast<long long>(blockIdx.x) * epi_threads + et; i < n4;
                 i += static_cast<long long>(gridDim.x) * epi_threads)
                o4[i] = z;
        }
        int it = 0;
        for (int t = first; t < num_tiles; t += step, ++it) {
            const Coord c = tile_coord(t, m_pairs, n_tiles);
            const int blk = 2 * c.m_blk + static_cast<int>(rank);
            if (kUp) {
                // cg 0: activation columns [0,64), cg 1: [64,128) of this CTA's 128 rows
                if (!warp_wait(sm.misc(0), it & 1, status, ST_TIMEOUT_TMEM_FULL, lane)) break;
                tc_fence_after();
                float g[64], u[64];
                ld32(g, tmem_addr(tmem_base, lane_base, cg * 64));
                ld32(g + 32, tmem_addr(tmem_base, lane_base, cg * 64 + 32));
                ld32(u, tmem_addr(tmem_base, lane_base, 128 + cg * 64));
                ld32(u + 32, tmem_addr(tmem_base, lane_base, 128 + cg * 64 + 32));
                tmem_ld_wait();
                tc_fence_before();
                warp_arrive_cluster(empty_leader, lane);   // accumulator drained: the next tile's main loop may start
#pragma unroll
                for (int i = 0; i < 64; ++i) g[i] = swiglu(g[i], u[i]);
                if (!warp_wait(sm.misc(3), (it & 1) ^ 1, status, ST_TIMEOUT_ACT, lane)) break;   // staging tile free
                uint8_t *sf_tile = a.act_sf + (static_cast<size_t>(blk) * n_tiles + c.n_tile) * SF_TILE;
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    float amax = 0.f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(g[q * 32 + i]));
                    float inv;
                    const uint32_t e = mx_block_scale(amax, &inv);
                    sf_tile[(row & 31) * 16 + (row >> 5) * 4 + cg * 2 + q] = static_cast<uint8_t>(e);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const float *v = g + q * 32 + j * 16;
                        const uint32_t chunk16 = static_cast<uint32_t>(cg * 4 + q * 2 + j);
                        st_shared_v4(sm.act + row * 128 + ((chunk16 ^ (row & 7)) << 4),
                                     pack_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv),
                                     pack_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv),
                                     pack_e4m3x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv),
                                     pack_e4m3x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv));
                    }
                }
                fence_proxy_async_smem();
                warp_arrive(sm.misc(2), lane);
                bool stored = true;
                if (et == 0) {
                    stored = mbar_wait(sm.misc(2), it & 1, status, ST_TIMEOUT_ACT);
                    if (stored) {
                        tma_store_2d(&map_act, sm.act, c.n_tile * 128, blk * BM);
                        tma_store_commit();
                        tma_store_wait_read<0>();
                        mbar_arrive(sm.misc(3));
                    }
                }
                if (!__shfl_sync(0xffffffffu, stored, 0)) break;   // keep the warp together on the error path
            } else {
                // cg selects output columns [cg*128, cg*128+128) of the 256-wide tile
                const int pair = a.sorted_ids[blk * BM + row];
                const int tok = pair >= 0 ? pair / a.top_k : 0;
                const bool valid = pair >= 0 && tok < a.M;
                const float wgt = valid ? a.topk_weights[pair] : 0.f;
                __nv_bfloat16 *dst = a.out + static_cast<size_t>(valid ? tok : 0) * a.K + c.n_tile * 256 + cg * 128;
                if (!warp_wait(sm.misc(0), it & 1, status, ST_TIMEOUT_TMEM_FULL, lane)) break;
                tc_fence_after();
                float v[128];
#pragma unroll
                for (int q = 0; q < 4; ++q) ld32(v + q * 32, tmem_addr(tmem_base, lane_base, cg * 128 + q * 32));
                tmem_ld_wait();
                tc_fence_before();
                warp_arrive_cluster(empty_leader, lane);
                if (a.bulk_reduce) {
                    const uint32_t red_row = sm.act + (threadIdx.x - 64) * RED_ROW_BYTES;
                    tma_store_wait_read<0>();
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        st_shared_v4(red_row + j * 16, pack_bf16x2(wgt * v[j * 8 + 0], wgt * v[j * 8 + 1]),
                                     pack_bf16x2(wgt * v[j * 8 + 2], wgt * v[j * 8 + 3]),
                                     pack_bf16x2(wgt * v[j * 8 + 4], wgt * v[j * 8 + 5]),
                                     pack_bf16x2(wgt * v[j * 8 + 6], wgt * v[j * 8 + 7]));
                    fence_proxy_async_smem();
                    if (valid) bulk_reduce_add_bf16(dst, red_row, 256);
                    tma_store_commit();
                    continue;
                }
                if (valid) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        red_add_bf16x8(dst + j * 8, pack_bf16x2(wgt * v[j * 8 + 0], wgt * v[j * 8 + 1]),
                                       pack_bf16x2(wgt * v[j * 8 + 2], wgt * v[j * 8 + 3]),
                                       pack_bf16x2(wgt * v[j * 8 + 4], wgt * v[j * 8 + 5]),
                                       pack_bf16x2(wgt * v[j * 8 + 6], wgt * v[j * 8 + 7]));
                }
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
// fused kernel (split == 0): per (row block, 128-wide H slice): gate/up GEMM -> SwiGLU -> MX requant ->
// e4m3 activation tile + its scale tile kept in shared memory -> down GEMM against w2[e][:, slice] in
// 128-column chunks -> weighted fp32 reductions into the zeroed fp32 buffer (split-K over H/128 slices).
//   TMEM: [0,256) gate|up accumulator, [256,384) scale regions, [384,512) down accumulator
//   misc barriers: 0 up_full | 1 up_empty | 2 act_ready | 3 act_free | 4 dn_full | 5 dn_empty
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS, 1)
moe_fused_mxfp8_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w1,
                       const __grid_constant__ CUtensorMap map_w2, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const Smem sm = carve(smem_raw, a.stages, ACT_EXTRA);
    const uint32_t act_sf_smem = sm.act + ACT_TILE_BYTES;
    int *status = &g_status_mxfp8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int epi_threads = EPI_WARPS * 32;
    constexpr uint32_t DN_ACC = 384;

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
        mbar_init(sm.misc(5), epi_threads);
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

    if (a.use_pdl) pdl_wait_primary();   // x_sorted / scale tiles come from the gather pre-pass

    const int m_blocks = live_row_blocks(a.npp, a.sorted_num);
    const int n_tiles = a.H / 128;
    const int num_tiles = m_blocks * n_tiles;
    const int ksteps = a.K / BKB;
    const int dn_chunks = a.K / 128;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            long long issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const Coord c = tile_coord(t, m_blocks, n_tiles);
                const int e = a.expert_ids[c.m_blk];
                const int row_gate = e * a.N + c.n_tile * 128;
                const int row_up = row_gate + a.H;
                const uint8_t *sf_gate = a.w_scales + static_cast<size_t>(row_gate >> 7) * ksteps * SF_TILE;
                const uint8_t *sf_up = a.w_scales + static_cast<size_t>(row_up >> 7) * ksteps * SF_TILE;
                const uint8_t *sf_x = a.xsf_tiles + static_cast<size_t>(c.m_blk) * ksteps * SF_TILE;
                for (int ks = 0; ks < ksteps; ++ks) {
                    ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_arrive_expect_tx(sm.full(s), STAGE_TX_BYTES);
                    tma_load_2d(sm.a(s), &map_x, sm.full(s), ks * BKB, c.m_blk * BM);
                    tma_load_2d(sm.b(s), &map_w1, sm.full(s), ks * BKB, row_gate);
                    tma_load_2d(sm.b(s) + B_BYTES / 2, &map_w1, sm.full(s), ks * BKB, row_up);
                    bulk_load_1d(sm.sfa(s), sf_x + static_cast<size_t>(ks) * SF_TILE, SF_TILE, sm.full(s));
                    bulk_load_1d(sm.sfb(s), sf_gate + static_cast<size_t>(ks) * SF_TILE, SF_TILE, sm.full(s));
                    bulk_load_1d(sm.sfb(s) + SF_TILE, sf_up + static_cast<size_t>(ks) * SF_TILE, SF_TILE, sm.full(s));
                    ++issued;
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (!ok) break;
                // down slots: 128 rows of w2[e] (output columns) x the 128 H-bytes of this slice + their scale tile
                const uint8_t *sf_w2 = a.w2_scales + (static_cast<size_t>(e) * (a.K / 128) * n_tiles + c.n_tile) * SF_TILE;
                for (int ch = 0; ch < dn_chunks; ++ch) {
                    ok = mbar_wait(sm.empty(s), ph ^ 1, status, ST_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_arrive_expect_tx(sm.full(s), B_BYTES / 2 + SF_TILE);
                    tma_load_2d(sm.b(s), &map_w2, sm.full(s), c.n_tile * 128, e * a.K + ch * 128);
                    bulk_load_1d(sm.sfb(s), sf_w2 + static_cast<size_t>(ch) * n_tiles * SF_TILE, SF_TILE, sm.full(s));
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
            constexpr uint32_t idesc_up = idesc_mxf8_f32(128, 256);
            constexpr uint32_t idesc_dn = idesc_mxf8_f32(128, 128);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            long long fill = 0, dn_it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
                ok = mbar_wait(sm.misc(1), (it & 1) ^ 1, status, ST_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                for (int ks = 0; ks < ksteps; ++ks, ++fill) {
                    ok = mbar_wait(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
                    issue_slot(tmem_base, sm.a(s), sm.b(s), sm.sfa(s), sm.sfb(s), sm.sfb(s) + SF_TILE, tmem_base, fill,
                               ks == 0, idesc_up, 2);
                    umma_commit(sm.empty(s));
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(sm.misc(0));
                ok = mbar_wait(sm.misc(2), it & 1, status, ST_TIMEOUT_ACT);
                if (!ok) break;
                tc_fence_after();
                for (int ch = 0; ch < dn_chunks; ++ch, ++fill, ++dn_it) {
                    ok = mbar_wait(sm.misc(5), static_cast<uint32_t>((dn_it & 1) ^ 1), status, ST_TIMEOUT_TMEM_EMPTY);
                    if (!ok) break;
                    ok = mbar_wait(sm.full(s), ph, status, ST_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
                    issue_slot(tmem_base + DN_ACC, sm.act, sm.b(s), act_sf_smem, sm.sfb(s), 0, tmem_base, fill, true,
                               idesc_dn, 1);
                    umma_commit(sm.empty(s));
                    umma_commit(sm.misc(4));
                    if (++s == a.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit(sm.misc(3));
            }
        }
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const uint32_t lane_base = (warp & 3) * 32;
        const int row = lane_base + lane;
        const int cg = ew >> 2;
        uint8_t *act_sf_generic = const_cast<uint8_t *>(smem_raw) + (act_sf_smem - smem_u32(smem_raw));
        int it = 0;
        long long dn_it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
            const Coord c = tile_coord(t, m_blocks, n_tiles);
            const int pair = a.sorted_ids[c.m_blk * BM + row];
            const int tok = pair >= 0 ? pair / a.top_k : 0;
            const bool valid = pair >= 0 && tok < a.M;
            const float wgt = valid ? a.topk_weights[pair] : 0.f;
            float *dst = a.acc32 + static_cast<size_t>(valid ? tok : 0) * a.K + cg * 64;
            if (!mbar_wait(sm.misc(0), it & 1, status, ST_TIMEOUT_TMEM_FULL)) break;
            tc_fence_after();
            {
                float g[64], u[64];
                ld32(g, tmem_addr(tmem_base, lane_base, cg * 64));
                ld32(g + 32, tmem_addr(tmem_base, lane_base, cg * 64 + 32));
                ld32(u, tmem_addr(tmem_base, lane_base, 128 + cg * 64));
                ld32(u + 32, tmem_addr(tmem_base, lane_base, 128 + cg * 64 + 32));
                tmem_ld_wait();
                tc_fence_before();
                mbar_arrive(sm.misc(1));
#pragma unroll
                for (int i = 0; i < 64; ++i) g[i] = swiglu(g[i], u[i]);
                if (!mbar_wait(sm.misc(3), (it & 1) ^ 1, status, ST_TIMEOUT_ACT)) break;   // act tile reusable
#pragma unroll
                for (int blk = 0; blk < 2; ++blk) {
                    float amax = 0.f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(g[blk * 32 + i]));
                    float inv;
                    const uint32_t e = mx_block_scale(amax, &inv);
                    act_sf_generic[(row & 31) * 16 + (row >> 5) * 4 + cg * 2 + blk] = static_cast<uint8_t>(e);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const float *v = g + blk * 32 + j * 16;
                        const uint32_t chunk16 = static_cast<uint32_t>(cg * 4 + blk * 2 + j);
                        st_shared_v4(sm.act + row * 128 + ((chunk16 ^ (row & 7)) << 4),
                                     pack_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv),
                                     pack_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv),
                                     pack_e4m3x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv),
                                     pack_e4m3x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv));
                    }
                }
                fence_proxy_async_smem();
                mbar_arrive(sm.misc(2));
            }
            for (int ch = 0; ch < dn_chunks; ++ch, ++dn_it) {
                ok = mbar_wait(sm.misc(4), static_cast<uint32_t>(dn_it & 1), status, ST_TIMEOUT_TMEM_FULL);
                if (!ok) break;
                tc_fence_after();
                float v[64];
                ld32(v, tmem_addr(tmem_base + DN_ACC, lane_base, cg * 64));
                ld32(v + 32, tmem_addr(tmem_base + DN_ACC, lane_base, cg * 64 + 32));
                tmem_ld_wait();
                tc_fence_before();
                mbar_arrive(sm.misc(5));
                if (valid) {
                    float *d = dst + ch * 128;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d + j * 4),
                                     "f"(wgt * v[j * 4 + 0]), "f"(wgt * v[j * 4 + 1]), "f"(wgt * v[j * 4 + 2]),
                                     "f"(wgt * v[j * 4 + 3])
                                     : "memory");
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// out[i] += bf16(acc32[i])
__global__ void __launch_bounds__(256)
finalize_acc32_mxfp8_kernel(const float *__restrict__ acc32, __nv_bfloat16 *__restrict__ out, long long n8,
                            int use_pdl) {
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
// host side
// ---------------------------------------------------------------------------------------------
struct Problem {
    const void *x, *x_scales, *w, *w_scales, *w2, *w2_scales;
    void *out;
    const int32_t *sorted_ids, *expert_ids, *npp;
    const float *topk_weights;
    int top_k, M, K, N, E, sorted_num, block_n, warp_n, stages, bpc, split;
};

int validate(const Problem &p, int block_m) {
    PMOE_REQUIRE(p.x && p.x_scales && p.w && p.w_scales && p.w2 && p.w2_scales && p.out && p.sorted_ids &&
                     p.expert_ids && p.npp && p.topk_weights,
                 PMOE_ERR_BAD_ARG, "fused_moe_mxfp8: null pointer");
    PMOE_REQUIRE(p.M > 0 && p.K > 0 && p.N > 0 && p.E > 0 && p.top_k > 0 && p.sorted_num >= 0, PMOE_ERR_BAD_ARG,
                 "fused_moe_mxfp8: M, K, N, num_experts, top_k must be positive");
    PMOE_REQUIRE((p.K & 255) == 0, PMOE_ERR_BAD_ARG, "K dimension must be a multiple of 256 on the mxfp8 path");
    PMOE_REQUIRE((p.N & 255) == 0, PMOE_ERR_BAD_ARG, "N dimension must be a multiple of 256 on the mxfp8 path");
    PMOE_REQUIRE((p.block_n == 64 && p.warp_n == 4) || (p.block_n == 32 && p.warp_n == 8), PMOE_ERR_UNSUPPORTED,
                 "(block_n, warp_n) must be (64, 4) or (32, 8)");
    PMOE_REQUIRE(p.stages > 0 && p.stages < 5, PMOE_ERR_UNSUPPORTED, "mxfp8 supports stages in 1..4");
    PMOE_REQUIRE(p.bpc == 1 || p.bpc == 2, PMOE_ERR_UNSUPPORTED, "bpc must be 1 or 2");
    PMOE_REQUIRE(p.bpc == 1 || p.split, PMOE_ERR_UNSUPPORTED, "bpc=2 (two-CTA MMA) requires split=True");
    PMOE_REQUIRE(p.bpc == 1 || p.sorted_num % 256 == 0, PMOE_ERR_BAD_ARG,
                 "bpc=2 requires routing tables built by moe_align with bpc=2 (rows padded to 256)");
    PMOE_REQUIRE(block_m == 128, PMOE_ERR_UNSUPPORTED, "Blackwell tcgen05 fused MoE requires block_m=128.");
    PMOE_REQUIRE(p.sorted_num % 128 == 0, PMOE_ERR_BAD_ARG, "sorted_num must be a multiple of block_m");
    PMOE_REQUIRE(static_cast<long long>(p.E) * p.N < (1ll << 31) && static_cast<long long>(p.E) * p.K < (1ll << 31),
                 PMOE_ERR_UNSUPPORTED, "E*N and E*K must fit in 31 bits");
    const uintptr_t align = reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.w) |
                            reinterpret_cast<uintptr_t>(p.w2) | reinterpret_cast<uintptr_t>(p.out) |
                            reinterpret_cast<uintptr_t>(p.w_scales) | reinterpret_cast<uintptr_t>(p.w2_scales) |
                            reinterpret_cast<uintptr_t>(p.sorted_ids);
    PMOE_REQUIRE((align & 15) == 0, PMOE_ERR_BAD_ARG,
                 "x, w, w2, out, w_scales, w2_scales and sorted_token_ids must be 16-byte aligned");
    return PMOE_OK;
}

template <typename Kernel>
int set_smem(Kernel k, size_t bytes) {
    PMOE_CUDA_OK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
    return PMOE_OK;
}

struct Workspace {
    size_t act_q, act_sf, acc32, x_sorted, xsf, total;
};
Workspace plan_workspace(int M, int K, int N, int sorted_num, int split) {
    Workspace w{};
    const size_t H = N / 2, blocks = sorted_num / BM;
    auto up = [](size_t v) { return (v + 1023) & ~static_cast<size_t>(1023); };
    if (!split) {   // fp32 accumulation buffer [M, K] instead of the activation workspace
        w.acc32 = 0;
        w.x_sorted = up(static_cast<size_t>(M) * K * sizeof(float));
        w.xsf = up(w.x_sorted + static_cast<size_t>(sorted_num) * K);
        w.total = up(w.xsf + blocks * (K / 128) * SF_TILE);
        return w;
    }
    w.act_q = 0;
    w.act_sf = up(w.act_q + static_cast<size_t>(sorted_num) * H);
    w.x_sorted = up(w.act_sf + blocks * (H / 128) * SF_TILE);
    w.xsf = up(w.x_sorted + static_cast<size_t>(sorted_num) * K);
    w.total = up(w.xsf + blocks * (K / 128) * SF_TILE);
    return w;
}

int run(const Problem &p, void *workspace, cudaStream_t stream) {
    const int H = p.N / 2;
    const int max_blocks = p.sorted_num / BM;
    if (max_blocks == 0) {
        if (p.split) PMOE_CUDA_OK(cudaMemsetAsync(p.out, 0, static_cast<size_t>(p.M) * p.K * 2, stream));
        return PMOE_OK;
    }
    Args a{};
    a.sorted_ids = p.sorted_ids;
    a.expert_ids = p.expert_ids;
    a.npp = p.npp;
    a.topk_weights = p.topk_weights;
    a.out = static_cast<__nv_bfloat16 *>(p.out);
    a.w_scales = static_cast<const uint8_t *>(p.w_scales);
    a.w2_scales = static_cast<const uint8_t *>(p.w2_scales);
    a.M = p.M;
    a.K = p.K;
    a.N = p.N;
    a.H = H;
    a.top_k = p.top_k;
    a.sorted_num = p.sorted_num;
    a.stages = std::min(p.stages, MAX_STAGES);
    a.live_rows = call_extras().live_rows;
    PMOE_REQUIRE(!call_extras().out_rows, PMOE_ERR_UNSUPPORTED, "fused_moe_mxfp8: out_rows is a bf16 split-pipeline option");
    const int sms = sm_count();
    const int phases = phase_mask();

    PMOE_REQUIRE(workspace && (reinterpret_cast<uintptr_t>(workspace) & 1023) == 0, PMOE_ERR_BAD_ARG,
                 "fused_moe_mxfp8: workspace must be 1024-byte aligned");
    const Workspace w = plan_workspace(p.M, p.K, p.N, p.sorted_num, p.split);
    uint8_t *base = static_cast<uint8_t *>(workspace);
    uint8_t *act_q = base + w.act_q, *act_sf = base + w.act_sf, *x_sorted = base + w.x_sorted, *xsf = base + w.xsf;
    a.act_sf = act_sf;
    a.xsf_tiles = xsf;
    a.acc32 = reinterpret_cast<float *>(base + w.acc32);

    CUtensorMap map_x, map_w1, map_act, map_w2;
    if (int rc = make_tmap_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x_sorted, p.sorted_num, p.K, 128, BKB,
                              CU_TENSOR_MAP_SWIZZLE_128B, "x_sorted"))
        return rc;
    if (int rc = make_tmap_2d(&map_w1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.w, static_cast<uint64_t>(p.E) * p.N, p.K,
                              128, BKB, CU_TENSOR_MAP_SWIZZLE_128B, "w"))
        return rc;
    if (int rc = make_tmap_2d(&map_act, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, act_q, p.sorted_num, H, 128, BKB,
                              CU_TENSOR_MAP_SWIZZLE_128B, "act"))
        return rc;
    if (int rc = make_tmap_2d(&map_w2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.w2, static_cast<uint64_t>(p.E) * p.K, H,
                              256, BKB, CU_TENSOR_MAP_SWIZZLE_128B, "w2"))
        return rc;
    CUtensorMap map_x_short, map_act_short;
    if (int rc = make_tmap_2d(&map_x_short, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x_sorted, p.sorted_num, p.K, SHORT_ROWS,
                              BKB, CU_TENSOR_MAP_SWIZZLE_128B, "x_sorted (short box)"))
        return rc;
    if (int rc = make_tmap_2d(&map_act_short, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, act_q, p.sorted_num, H, SHORT_ROWS,
                              BKB, CU_TENSOR_MAP_SWIZZLE_128B, "act (short box)"))
        return rc;
    a.short_boxes = short_boxes_mode();

    // In-kernel row gather for the one-CTA gate/up kernel (PMOE_AGATHER=lsu): the pre-pass (routed rows written and
    // read again, scale rows re-tiled) disappears, but unlike bf16 it does not pay here - the gate/up kernel gets
    // 10-18 % slower with the four gather warps beside its eight epilogue warps (c2 T=8192 247 -> 292 us, c3 4.82 ->
    // 5.30 ms, c4 6.72 -> 7.94 ms), more than the pre-pass costs (37 us, 0.34 ms, 0.82 ms) except on c3 (-1 %). So the
    // pre-pass stays the default and the gather an option.
    const int a_mode = a_operand_mode();
    const bool lsu = p.split && p.bpc == 1 && a_mode == 2 && (reinterpret_cast<uintptr_t>(p.x_scales) & 3) == 0;
    if ((phases & 1) && !lsu) {
        gather_rows_mxfp8_kernel<<<std::min(4 * sms, (p.sorted_num + 7) / 8), 256, 0, stream>>>(
            static_cast<const uint8_t *>(p.x), static_cast<const uint8_t *>(p.x_scales), x_sorted, xsf, a);
        PMOE_CUDA_OK(cudaGetLastError());
    }
    if (!p.split) {
        // memset(acc32) -> [gather] -> fused kernel -> out += bf16(acc32)
        CUtensorMap map_w2f;
        if (int rc = make_tmap_2d(&map_w2f, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.w2, static_cast<uint64_t>(p.E) * p.K,
                                  H, 128, BKB, CU_TENSOR_MAP_SWIZZLE_128B, "w2"))
            return rc;
        const size_t elems = static_cast<size_t>(p.M) * p.K;
        PMOE_CUDA_OK(cudaMemsetAsync(a.acc32, 0, elems * sizeof(float), stream));
        const int use_pdl = pdl_enabled() ? 1 : 0;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        {
            Args fa = a;
            fa.use_pdl = use_pdl;
            const size_t smem = smem_bytes(fa.stages, ACT_EXTRA);
            if (int rc = set_smem(moe_fused_mxfp8_kernel, smem)) return rc;
            const int tiles = max_blocks * (H / 128);
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(std::min(tiles, sms));
            cfg.blockDim = dim3(THREADS);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = stream;
            cfg.attrs = attr;
            cfg.numAttrs = use_pdl ? 1 : 0;
            PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, moe_fused_mxfp8_kernel, map_x, map_w1, map_w2f, fa));
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(std::min<size_t>(4 * sms, (elems / 8 + 255) / 256)));
        cfg.blockDim = dim3(256);
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = use_pdl ? 1 : 0;
        PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, finalize_acc32_mxfp8_kernel, static_cast<const float *>(a.acc32), a.out,
                                        static_cast<long long>(elems / 8), use_pdl));
        return PMOE_OK;
    }
    if (p.bpc == 2) {
        // CTA pairs: B tiles travel as 128-row halves, the 512-byte scale tiles as rows of 128 32-bit words
        CUtensorMap map_w2h, sf_x, sf_w1, sf_act, sf_w2;
        if (int rc = make_tmap_2d(&map_w2h, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.w2, static_cast<uint64_t>(p.E) * p.K,
                                  H, 128, BKB, CU_TENSOR_MAP_SWIZZLE_128B, "w2 (half tiles)"))
            return rc;
        const uint64_t kt = p.K / 128, ht = H / 128;
        if (int rc = make_tmap_2d(&sf_x, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, xsf, max_blocks * kt, 128, 1, 128,
                                  CU_TENSOR_MAP_SWIZZLE_NONE, "x scale tiles"))
            return rc;
        if (int rc = make_tmap_2d(&sf_w1, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, p.w_scales,
                                  static_cast<uint64_t>(p.E) * p.N / 128 * kt, 128, 1, 128, CU_TENSOR_MAP_SWIZZLE_NONE,
                                  "w scale tiles"))
            return rc;
        if (int rc = make_tmap_2d(&sf_act, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, act_sf, max_blocks * ht, 128, 1, 128,
                                  CU_TENSOR_MAP_SWIZZLE_NONE, "activation scale tiles"))
            return rc;
        if (int rc = make_tmap_2d(&sf_w2, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, p.w2_scales,
                                  static_cast<uint64_t>(p.E) * p.K / 128 * ht, 128, 1, 128, CU_TENSOR_MAP_SWIZZLE_NONE,
                                  "w2 scale tiles"))
            return rc;
        PMOE_REQUIRE((reinterpret_cast<uintptr_t>(p.w_scales) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.w2_scales) & 15) == 0,
                     PMOE_ERR_BAD_ARG, "fused_moe_mxfp8: packed scales must be 16-byte aligned");
        Args pa = a;
        pa.stages = std::min(PAIR_MAX_STAGES, (a.stages * 3 + 1) / 2);   // same ring bytes as the 1-CTA kernels
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        auto launch_pair = [&](auto kernel, const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &msa,
                               const CUtensorMap &msb, const Args &args, int tiles, uint32_t extra, int nattr) -> int {
            const size_t smem = smem_bytes_pair(args.stages, extra);
            if (int rc = set_smem(kernel, smem)) return rc;
            PMOE_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 0));
            cudaLaunchConfig_t cfg = {};
            cfg.blockDim = dim3(THREADS);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = stream;
            cfg.attrs = attr;
            cfg.numAttrs = nattr;
            cfg.gridDim = dim3(2);
            int max_clusters = 0;
            PMOE_CUDA_OK(cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg));
            if (max_clusters < 1) return set_error(PMOE_ERR_CUDA, "no CTA pair of the bpc=2 kernel fits on this device");
            cfg.gridDim = dim3(2 * std::min(tiles, max_clusters));
            PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, ma, mb, msa, msb, map_act, args));
            return PMOE_OK;
        };
        if (phases & 2) {
            Args up = pa;
            up.zero_out = 1;
            up.use_pdl = (pdl_enabled() && (phases & 1)) ? 1 : 0;
            if (int rc = launch_pair(moe_pair_mxfp8_kernel<true>, map_x, map_w1, sf_x, sf_w1, up,
                                     (max_blocks / 2) * (H / 128), ACT_EXTRA, up.use_pdl ? 2 : 1))
                return rc;
        }
        if (phases & 4) {
            Args dn = pa;
            dn.use_pdl = (pdl_enabled() && (phases & 2)) ? 1 : 0;
            const int bulk = down_bulk_reduce_mode();
            dn.bulk_reduce = (bulk < 0 ? (H <= 1024) : bulk != 0) ? 1 : 0;
            if (dn.bulk_reduce) dn.stages = std::min(dn.stages, 4);   // room for the reduction staging tile
            if (int rc = launch_pair(moe_pair_mxfp8_kernel<false>, map_act, map_w2h, sf_act, sf_w2, dn,
                                     (max_blocks / 2) * (p.K / 256), dn.bulk_reduce ? RED_STAGE_BYTES : 0u,
                                     dn.use_pdl ? 2 : 1))
                return rc;
        }
        return PMOE_OK;
    }
    if (phases & 2) {
        Args up = a;
        up.zero_out = 1;
        up.lsu_gather = lsu ? 1 : 0;
        up.x = static_cast<const uint8_t *>(p.x);
        up.x_scales = static_cast<const uint8_t *>(p.x_scales);
        const size_t smem = smem_bytes(up.stages, ACT_EXTRA);
        if (int rc = set_smem(moe_up_mxfp8_kernel, smem)) return rc;
        const int tiles = max_blocks * (H / 128);
        up.use_pdl = (pdl_enabled() && (phases & 1) && !lsu) ? 1 : 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(std::min(tiles, sms));
        cfg.blockDim = dim3(lsu ? UP_MAX_THREADS : THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = up.use_pdl ? 1 : 0;
        PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, moe_up_mxfp8_kernel, map_x, map_w1, map_act, map_x_short, map_act_short, up));
    }
    if (phases & 4) {
        Args dn = a;
        dn.use_pdl = (pdl_enabled() && (phases & 2)) ? 1 : 0;
        const int bulk = down_bulk_reduce_mode();   // -1 auto: on when the down GEMM's K extent (H) is short
        dn.bulk_reduce = (bulk < 0 ? (H <= 1024) : bulk != 0) ? 1 : 0;
        if (dn.bulk_reduce) dn.stages = std::min(dn.stages, 3);   // room for the reduction staging tile
        const size_t smem = smem_bytes(dn.stages, dn.bulk_reduce ? RED_STAGE_BYTES : 0u);
        if (int rc = set_smem(moe_down_mxfp8_kernel, smem)) return rc;
        const int tiles = max_blocks * (p.K / 256);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(std::min(tiles, sms));
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = dn.use_pdl ? 1 : 0;
        PMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, moe_down_mxfp8_kernel, map_act, map_w2, map_act_short, dn));
    }
    return PMOE_OK;
}

}  // namespace

int wait_ns_store_mxfp8(unsigned long long ns) {
    PMOE_CUDA_OK(cudaMemcpyToSymbol(g_wait_ns, &ns, sizeof(ns)));
    return PMOE_OK;
}

int status_fetch_mxfp8(int *value, bool reset) {
    if (value) PMOE_CUDA_OK(cudaMemcpyFromSymbol(value, g_status_mxfp8, sizeof(int)));
    if (reset) {
        const int zero = 0;
        PMOE_CUDA_OK(cudaMemcpyToSymbol(g_status_mxfp8, &zero, sizeof(int)));
    }
    return PMOE_OK;
}

}  // namespace pmoe

extern "C" size_t pmoe_fused_moe_mxfp8_workspace_bytes(int M, int K, int N, int sorted_num, int split) {
    if (sorted_num <= 0 || N <= 0 || K <= 0) return 0;
    return pmoe::plan_workspace(M, K, N, sorted_num, split).total;
}

extern "C" int pmoe_fused_moe_mxfp8_ws(const void *x, const void *x_scales, const void *w, const void *w_scales,
                                       const void *w2, const void *w2_scales, void *out,
                                       const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                       const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k,
                                       int M, int K, int N, int num_experts, int sorted_num, int block_m,
                                       int block_n, int warp_n, int stages, int bpc, int split, void *workspace,
                                       size_t workspace_bytes, pmoe_stream_t stream) {
    using namespace pmoe;
    Problem p{x, x_scales, w, w_scales, w2, w2_scales, out, sorted_token_ids, expert_ids, num_tokens_post_padded,
              topk_weights, top_k, M, K, N, num_experts, sorted_num, block_n, warp_n, stages, bpc, split ? 1 : 0};
    if (int rc = validate(p, block_m)) return rc;
    const size_t need = pmoe_fused_moe_mxfp8_workspace_bytes(M, K, N, sorted_num, split);
    PMOE_REQUIRE(need == 0 || (workspace && workspace_bytes >= need), PMOE_ERR_BAD_ARG,
                 "fused_moe_mxfp8: workspace of %zu bytes required, got %zu", need, workspace_bytes);
    return run(p, workspace, stream);
}

extern "C" int pmoe_fused_moe_mxfp8(const void *x, const void *x_scales, const void *w, const void *w_scales,
                                    const void *w2, const void *w2_scales, void *out,
                                    const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                    const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k, int M,
                                    int K, int N, int num_experts, int sorted_num, int block_m, int block_n,
                                    int warp_n, int stages, int bpc, int split, pmoe_stream_t stream) {
    using namespace pmoe;
    Problem p{x, x_scales, w, w_scales, w2, w2_scales, out, sorted_token_ids, expert_ids, num_tokens_post_padded,
              topk_weights, top_k, M, K, N, num_experts, sorted_num, block_n, warp_n, stages, bpc, split ? 1 : 0};
    if (int rc = validate(p, block_m)) return rc;
    const size_t need = pmoe_fused_moe_mxfp8_workspace_bytes(M, K, N, sorted_num, split);
    void *raw = nullptr;
    if (need)
        if (int rc = scratch_alloc(&raw, need + 1024, stream)) return rc;
    void *ws = reinterpret_cast<void *>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int rc = run(p, raw ? ws : nullptr, stream);
    if (raw)
        if (int rc2 = scratch_free(raw, stream)) return rc2;
    return rc;
}

extern "C" int pmoe_fused_moe_mxfp8_ex(const void *x, const void *x_scales, const void *w, const void *w_scales,
                                       const void *w2, const void *w2_scales, void *out,
                                       const int32_t *sorted_token_ids, const int32_t *expert_ids,
                                       const int32_t *num_tokens_post_padded, const float *topk_weights, int top_k,
                                       int M, int K, int N, int num_experts, int sorted_num, int block_m, int block_n,
                                       int warp_n, int stages, int bpc, int split, void *workspace,
                                       size_t workspace_bytes, const int32_t *live_rows, pmoe_stream_t stream) {
    pmoe::CallExtras &extras = pmoe::call_extras();
    extras.live_rows = live_rows;
    const int rc = pmoe_fused_moe_mxfp8_ws(x, x_scales, w, w_scales, w2, w2_scales, out, sorted_token_ids, expert_ids,
                                           num_tokens_post_padded, topk_weights, top_k, M, K, N, num_experts, sorted_num,
                                           block_m, block_n, warp_n, stages, bpc, split, workspace, workspace_bytes,
                                           stream);
    extras = pmoe::CallExtras{};
    return rc;
}
