// Host-side plumbing behind the C ABI: error string, tensor-map encoder lookup, device queries,
// device status read-back.
#include "host_common.h"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cudaTypedefs.h>

#include <mutex>

#include "ptx.cuh"

namespace pmoe {

// status word of the kernels of this translation unit (the wait probe)
__device__ int g_status_misc = 0;

// One CTA, one thread: waits on an mbarrier that nothing ever arrives on, so the bounded wait runs out after
// the current limit (pmoe_debug_set_wait_ns), records ST_TIMEOUT_PROBE and the kernel ends through its normal
// exit. Exercises exactly the wait every GEMM kernel of this library uses, without involving one.
__global__ void wait_probe_kernel() {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
        (void)mbar_wait(smem_u32(&bar), 0, &g_status_misc, ST_TIMEOUT_PROBE);
    }
}

namespace {
thread_local char g_error[512] = "";
std::once_flag g_encode_once;
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
    std::call_once(g_encode_once, [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    });
    return g_encode;
}
}  // namespace

CallExtras &call_extras() {
    thread_local CallExtras extras;
    return extras;
}

int set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int make_tmap_2d(CUtensorMap *map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void *base,
                 uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols,
                 CUtensorMapSwizzle swizzle, const char *what) {
    auto encode = tensor_map_encoder();
    PMOE_REQUIRE(encode != nullptr, PMOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * elem_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(map, dtype, 2, const_cast<void *>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    PMOE_REQUIRE(r == CUDA_SUCCESS, PMOE_ERR_CUDA,
                 "tensor map '%s' (rows %llu, cols %llu, box %ux%u) failed: CUresult %d", what,
                 static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols), box_rows, box_cols,
                 static_cast<int>(r));
    return PMOE_OK;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// One private stream-ordered memory pool per device, created on first use, with the release threshold
// raised so that freed scratch stays cached in the pool instead of going back to the driver at every
// synchronisation (the default pool's threshold is 0, which makes each malloc cost ~0.2 ms).
int scratch_alloc(void **ptr, size_t bytes, cudaStream_t stream) {
    static cudaMemPool_t pools[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    PMOE_CUDA_OK(cudaGetDevice(&dev));
    PMOE_REQUIRE(dev >= 0 && dev < 64, PMOE_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!pools[dev]) {
            cudaMemPoolProps props = {};
            props.allocType = cudaMemAllocationTypePinned;
            props.location.type = cudaMemLocationTypeDevice;
            props.location.id = dev;
            PMOE_CUDA_OK(cudaMemPoolCreate(&pools[dev], &props));
            unsigned long long keep = ~0ull;
            PMOE_CUDA_OK(cudaMemPoolSetAttribute(pools[dev], cudaMemPoolAttrReleaseThreshold, &keep));
        }
    }
    PMOE_CUDA_OK(cudaMallocFromPoolAsync(ptr, bytes, pools[dev], stream));
    return PMOE_OK;
}

int scratch_free(void *ptr, cudaStream_t stream) {
    PMOE_CUDA_OK(cudaFreeAsync(ptr, stream));
    return PMOE_OK;
}

bool pdl_enabled() {
    static const bool on = [] {
        const char *e = getenv("PMOE_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

int a_operand_mode() {   // read on every call: tests switch modes inside one process
    const char *e = getenv("PMOE_AGATHER");
    if (e && !strcmp(e, "tma4")) return 0;
    if (e && !strcmp(e, "lsu")) return 2;
    if (e && !strcmp(e, "pre")) return 1;
    if (getenv("PMOE_PREGATHER")) return pregather_enabled() ? 1 : 0;
    return -1;   // auto: chosen per call from the layer width and the routed rows per expert
}

int down_bulk_reduce_mode() {   // read on every call: tests switch modes inside one process
    const char *e = getenv("PMOE_DOWN_BULK");
    return e ? (e[0] == '0' ? 0 : 1) : -1;
}

static int g_l2_ahead = -1;
int l2_prefetch_distance() {
    if (g_l2_ahead < 0) {
        const char *e = getenv("PMOE_L2_AHEAD");
        const int v = e ? atoi(e) : 0;
        g_l2_ahead = v < 0 ? 0 : (v > 64 ? 64 : v);
    }
    return g_l2_ahead;
}

int dual_blocks_mode() {
    const char *e = getenv("PMOE_DUAL");
    return e ? (e[0] == '0' ? 0 : 1) : -1;
}

bool pair_tails_enabled() {
    const char *e = getenv("PMOE_PAIR_TAILS");   // read on every call: tests compare both settings
    return !(e && e[0] == '0');
}

int short_boxes_mode() {
    const char *e = getenv("PMOE_SHORT_A");
    return e ? atoi(e) & 3 : 3;
}

static int g_phase_mask = 7;
int phase_mask() { return g_phase_mask; }

bool pregather_enabled() {   // read on every call, like the other per-call switches
    const char *e = getenv("PMOE_PREGATHER");
    return !(e && e[0] == '0');
}

int status_fetch_bf16(int *value, bool reset);
int status_fetch_mxfp8(int *value, bool reset);
int status_fetch_ep(int *value, bool reset);
int status_fetch_bwd(int *value, bool reset);
int wait_ns_store_bwd(unsigned long long ns);
int wait_ns_store_ep(unsigned long long ns);
int wait_ns_store_bf16(unsigned long long ns);
int wait_ns_store_mxfp8(unsigned long long ns);

static int status_fetch_misc(int *value, bool reset) {
    if (value) PMOE_CUDA_OK(cudaMemcpyFromSymbol(value, g_status_misc, sizeof(int)));
    if (reset) {
        const int zero = 0;
        PMOE_CUDA_OK(cudaMemcpyToSymbol(g_status_misc, &zero, sizeof(int)));
    }
    return PMOE_OK;
}

}  // namespace pmoe

extern "C" const char *pmoe_last_error(void) { return pmoe::g_error; }

extern "C" int pmoe_version(void) { return 100; }

extern "C" int pmoe_debug_set_l2_ahead(int ksteps) {
    const int old = pmoe::l2_prefetch_distance();
    pmoe::g_l2_ahead = ksteps < 0 ? 0 : (ksteps > 64 ? 64 : ksteps);
    return old;
}

extern "C" int pmoe_debug_set_phase_mask(int mask) {
    const int old = pmoe::g_phase_mask;
    pmoe::g_phase_mask = mask & 15;
    return old;
}

extern "C" int pmoe_device_status(int *status) {
    using namespace pmoe;
    PMOE_REQUIRE(status != nullptr, PMOE_ERR_BAD_ARG, "pmoe_device_status: null pointer");
    PMOE_CUDA_OK(cudaDeviceSynchronize());
    int a = 0, b = 0, c = 0, d = 0, e = 0;
    if (int rc = status_fetch_bf16(&a, false)) return rc;
    if (int rc = status_fetch_bwd(&e, false)) return rc;
    if (int rc = status_fetch_mxfp8(&b, false)) return rc;
    if (int rc = status_fetch_misc(&c, false)) return rc;
    if (int rc = status_fetch_ep(&d, false)) return rc;
    *status = a ? a : (b ? b : (c ? c : (d ? d : e)));
    if (*status) return set_error(PMOE_ERR_DEVICE, "a kernel gave up a bounded wait (device status %d)", *status);
    return PMOE_OK;
}

extern "C" int pmoe_reset_device_status(void) {
    using namespace pmoe;
    PMOE_CUDA_OK(cudaDeviceSynchronize());
    if (int rc = status_fetch_bf16(nullptr, true)) return rc;
    if (int rc = status_fetch_mxfp8(nullptr, true)) return rc;
    if (int rc = status_fetch_ep(nullptr, true)) return rc;
    if (int rc = status_fetch_bwd(nullptr, true)) return rc;
    return status_fetch_misc(nullptr, true);
}

extern "C" int pmoe_debug_set_wait_ns(unsigned long long ns) {
    using namespace pmoe;
    PMOE_REQUIRE(ns >= 1000ull && ns <= 60000000000ull, PMOE_ERR_BAD_ARG,
                 "pmoe_debug_set_wait_ns: the limit must lie between 1 microsecond and 60 seconds");
    if (int rc = wait_ns_store_bf16(ns)) return rc;
    if (int rc = wait_ns_store_mxfp8(ns)) return rc;
    if (int rc = wait_ns_store_ep(ns)) return rc;
    if (int rc = wait_ns_store_bwd(ns)) return rc;
    PMOE_CUDA_OK(cudaMemcpyToSymbol(g_wait_ns, &ns, sizeof(ns)));
    return PMOE_OK;
}

extern "C" int pmoe_debug_wait_probe(pmoe_stream_t stream) {
    using namespace pmoe;
    wait_probe_kernel<<<1, 32, 0, stream>>>();
    PMOE_CUDA_OK(cudaGetLastError());
    return PMOE_OK;
}
