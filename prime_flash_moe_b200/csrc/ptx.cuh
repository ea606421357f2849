// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (MMA, TMEM
// alloc/load, commit) and the shared-memory / instruction descriptor encoders used by every GEMM
// kernel of this library.
//
// Every wait in this file is bounded: a wait that does not complete within PMOE_WAIT_NS records an
// error code in a device status word and returns false, and the caller unwinds to the kernel's
// common teardown (TMEM dealloc, exit). A kernel of this library therefore never spins forever.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pmoe {

// ---------------------------------------------------------------------------------------------
// status word
// ---------------------------------------------------------------------------------------------
// Device status codes (0 = ok). The first failing wait wins (atomicCAS from 0).
enum : int {
    ST_OK = 0,
    ST_TIMEOUT_EMPTY = 1,       // producer waited for a free ring slot
    ST_TIMEOUT_FULL = 2,        // MMA issuer waited for a filled ring slot
    ST_TIMEOUT_TMEM_EMPTY = 3,  // MMA issuer waited for a drained accumulator
    ST_TIMEOUT_TMEM_FULL = 4,   // epilogue waited for a finished accumulator
    ST_TIMEOUT_ACT = 5,         // fused kernel: wait on the on-chip activation tile hand-off
    ST_TIMEOUT_DRAIN = 6,       // teardown waited for copies in flight
    ST_TIMEOUT_PEER = 7,        // 2-CTA kernels: wait on the peer CTA
    ST_TIMEOUT_PROBE = 9,       // the wait-probe kernel waited on a barrier nobody arrives on (8 = bad CTA pair)
};

#ifndef PMOE_WAIT_NS
#define PMOE_WAIT_NS 2000000000ull  // 2 s per wait
#endif

// Limit of every bounded wait in nanoseconds. One copy per translation unit (no relocatable device code);
// pmoe_debug_set_wait_ns() stores the same value into all of them on the current device.
static __device__ unsigned long long g_wait_ns = PMOE_WAIT_NS;
__device__ __forceinline__ unsigned long long wait_limit_ns() {
    return *reinterpret_cast<volatile unsigned long long *>(&g_wait_ns);
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// one elected lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// generic-proxy writes to shared memory -> visible to the async proxy (TMA store, tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait. Returns false if the wait gave up (own time-out, or another thread of the grid
// already recorded an error); the status word then holds the first error code.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, int *status, int code) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t n = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++n & 63u) == 0) {
            if (*reinterpret_cast<volatile int *>(status) != 0) return false;
            if (globaltimer_ns() - t0 > wait_limit_ns()) {
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int *status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, status, code);
}

// ---------------------------------------------------------------------------------------------
// TMA
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0,
                                            int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0,
                                            int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// pull one box of a 2-D tensor from HBM into L2 (no shared-memory destination, no completion signal)
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap *map, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1)
                 : "memory");
}
// four rows r0..r3 of a 2-D tensor, `box[0]` columns starting at `col`, land as four consecutive
// rows at dst (the tensor map's box is {cols, 1})
__device__ __forceinline__ void tma_gather4(uint32_t dst, const CUtensorMap *map, uint32_t bar, int col,
                                            int r0, int r1, int r2, int r3) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
        : "memory");
}
// untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16)
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1)
                 : "memory");
}
// global[dst .. dst+bytes) += shared[src .. src+bytes) element-wise in bf16 (one bulk reduction handled
// by the TMA engine; both addresses 16-byte aligned, bytes a multiple of 16; joins the thread's bulk group)
__device__ __forceinline__ void bulk_reduce_add_bf16(void *gdst, uint32_t ssrc, uint32_t bytes) {
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.bf16 [%0], [%1], %2;"
                 ::"l"(gdst), "r"(ssrc), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the N most recent groups have finished READING shared memory
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// all but the N most recent groups are complete (writes performed)
template <int N>
__device__ __forceinline__ void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------------
// LSU-side asynchronous copies (row gathers the TMA engine is too slow for)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
// the barrier receives one (pre-counted) arrival once all earlier cp.async of this thread have landed
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// programmatic dependent launch
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait_primary() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: TMEM management
// ---------------------------------------------------------------------------------------------
// whole warp; writes the TMEM base address to *dst_smem
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
    return base + (lane << 16) + col;
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp receives lane (addr.lane + i), 32 columns
__device__ __forceinline__ void tmem_ld_32x32(float (&d)[32], uint32_t addr) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]), "=f"(d[4]), "=f"(d[5]), "=f"(d[6]), "=f"(d[7]),
          "=f"(d[8]), "=f"(d[9]), "=f"(d[10]), "=f"(d[11]), "=f"(d[12]), "=f"(d[13]), "=f"(d[14]),
          "=f"(d[15]), "=f"(d[16]), "=f"(d[17]), "=f"(d[18]), "=f"(d[19]), "=f"(d[20]), "=f"(d[21]),
          "=f"(d[22]), "=f"(d[23]), "=f"(d[24]), "=f"(d[25]), "=f"(d[26]), "=f"(d[27]), "=f"(d[28]),
          "=f"(d[29]), "=f"(d[30]), "=f"(d[31])
        : "r"(addr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// tcgen05: descriptors
// ---------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major operand tile written by TMA with SWIZZLE_128B:
// rows are 128 B apart, 8-row groups (1024 B) repeat with stride SBO = 1024 B. The tile base must be
// 1024-B aligned; stepping along K inside the 128-B row is done by adding the byte offset to `addr`.
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4 (unused here)
//   bits 32-45 stride byte offset >> 4 bits 46-47 descriptor version (1 on sm_100)
//   bits 61-63 layout: 0 none, 2 = 128 B swizzle, 4 = 64 B, 6 = 32 B
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}

// Shared-memory descriptor of one 512-byte scale-factor tile (32 lines of 16 bytes, no swizzle) for
// tcgen05.cp.32x128b: four 8-line core matrices 128 bytes apart (SBO = 128).
__device__ __forceinline__ uint64_t smem_desc_sf(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(128 >> 4) << 32) | (1ull << 46);
}

// Instruction descriptor, kind::f16, bf16 x bf16 -> fp32, both operands K-major.
//   bits 4-5 D format (1 = f32), 7-9 A format (1 = bf16), 10-12 B format, 15/16 A/B major (0 = K),
//   bits 17-22 N >> 3, bits 24-28 M >> 4
__host__ __device__ constexpr uint32_t idesc_bf16_f32(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Instruction descriptor, kind::mxf8f6f4.block_scale, e4m3 x e4m3 -> fp32 with ue8m0 scales
// (one scale per 32 K-elements), K-major operands, MMA-K = 32.
//   bits 4-5 B scale-factor id, 7-9 A format (0 = e4m3), 10-12 B format, 17-22 N >> 3,
//   bit 23 scale format (1 = ue8m0), 24-28 M >> 4, 29-30 A scale-factor id
__host__ __device__ constexpr uint32_t idesc_mxf8_f32(uint32_t m, uint32_t n) {
    return ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24);
}
__host__ __device__ constexpr uint32_t idesc_with_sf_ids(uint32_t idesc, uint32_t a_sf_id, uint32_t b_sf_id) {
    return (idesc & ~((3u << 4) | (3u << 29))) | ((b_sf_id & 3u) << 4) | ((a_sf_id & 3u) << 29);
}

// ---------------------------------------------------------------------------------------------
// tcgen05: MMA issue (one thread), commit
// ---------------------------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]^T ; M = 128 (cta_group::1)
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
// scale factors: 32 lanes x 128 bit from shared memory, replicated to the four 32-lane quarters
__device__ __forceinline__ void tmem_cp_sf_32x128b_warpx4(uint32_t dst_tmem, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(dst_tmem), "l"(sdesc) : "memory");
}
// the mbarrier receives one arrival when every previously issued tcgen05 op of this thread is done
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// ---------------------------------------------------------------------------------------------
// CTA pairs (cluster of 2, tcgen05 cta_group::2): the even CTA of the pair issues the MMAs, each CTA
// loads its own half of the operands and owns the accumulator rows of its half of M
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait on a barrier whose arrivals may come from the peer CTA
static __device__ __noinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int *status, int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t n = 0;
    while (!mbar_try_wait_cluster(bar, parity)) {
        if ((++n & 63u) == 0) {
            if (*reinterpret_cast<volatile int *>(status) != 0) return false;
            if (globaltimer_ns() - t0 > wait_limit_ns()) {
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
    return true;
}
// tile load whose completion bytes are signalled on `bar_cluster_addr`, which may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}
// one warp of EACH CTA of the pair executes these
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B^T with M = 256 (128 rows per CTA), B rows split between the CTAs
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// block-scaled e4m3 x e4m3 version: A/B halves and the scale factors are read from each CTA's own shared
// memory / tensor memory at the same offsets
__device__ __forceinline__ void umma_mxf8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
// scale-factor copy executed for both CTAs of the pair (each from its own shared memory into its own TMEM)
__device__ __forceinline__ void tmem_cp_sf_32x128b_warpx4_pair(uint32_t dst_tmem, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(dst_tmem), "l"(sdesc) : "memory");
}
// one arrival on the barrier at the same shared-memory offset in every CTA of `cta_mask`
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask)
                 : "memory");
}

// ---------------------------------------------------------------------------------------------
// misc
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
// out[0..8) += v (bf16x2 vector reduction, relaxed, no return value)
__device__ __forceinline__ void red_add_bf16x8(__nv_bfloat16 *dst, uint32_t a, uint32_t b, uint32_t c,
                                               uint32_t d) {
    asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(a), "r"(b), "r"(c),
                 "r"(d)
                 : "memory");
}
// eight 32-bit words (32 bytes, one whole sector) to global memory in one instruction; `dst` 32-byte aligned
__device__ __forceinline__ void st_global_v8(void *dst, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}
__device__ __forceinline__ void ld_global_v8(const void *src, uint32_t (&w)[8]) {
    asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "l"(src)
                 : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// SwiGLU on fp32 accumulators: up * silu(gate). The quotient is the approximate division (2 ulp): the IEEE
// one branches into a slow path when the denominator leaves [2^-126, 2^126], which padding rows (whose
// accumulators are arbitrary bit patterns) hit all the time - it made the gate/up epilogue several times slower.
__device__ __forceinline__ float swiglu(float gate, float up) {
    return up * __fdividef(gate, 1.f + __expf(-gate));
}

}  // namespace pmoe
