// Host-side helpers shared by the translation units behind the C ABI: status codes, the
// thread-local error string, CUDA error mapping and the driver entry point for tensor maps.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pmoe_b200.h"

namespace pmoe {

// stores a printf-formatted message for pmoe_last_error() and returns `code`
int set_error(int code, const char *fmt, ...);

#define PMOE_CUDA_OK(expr)                                                                          \
    do {                                                                                            \
        cudaError_t _e = (expr);                                                                    \
        if (_e != cudaSuccess)                                                                      \
            return ::pmoe::set_error(PMOE_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                 \
                                     cudaGetErrorString(_e), __FILE__, __LINE__);                   \
    } while (0)

#define PMOE_REQUIRE(cond, code, ...)                                 \
    do {                                                              \
        if (!(cond)) return ::pmoe::set_error(code, __VA_ARGS__);     \
    } while (0)

// 2-D row-major tensor map: `rows` x `cols` elements of `elem_bytes` each, row pitch = cols*elem_bytes,
// box = box_rows x box_cols, given swizzle. Returns PMOE_OK or an error code.
int make_tmap_2d(CUtensorMap *map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void *base,
                 uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols,
                 CUtensorMapSwizzle swizzle, const char *what);

// stream-ordered scratch from a private per-device pool (used by the entry points without `_ws`)
int scratch_alloc(void **ptr, size_t bytes, cudaStream_t stream);
int scratch_free(void *ptr, cudaStream_t stream);

// Optional extras of one call, set by the `_ex` entry points around the regular launch path (thread-local):
//   live_rows  device int32[1]: only rows below *live_rows of `out` (and of x) are in use - the launchers then zero
//              only those rows of `out`
//   out_rows   device uint64[M]: row i of `out` lives at this address (possibly in another GPU's memory mapped
//              into this process); the down kernels add their results there with plain vector reductions and the
//              library does not zero anything (bf16 split pipeline only)
//   gu_out     device bf16[sorted_num, N]: the gate/up kernel also stores its pre-activations there (kept for the
//              backward pass; bf16 split pipeline with bpc = 1 only)
struct CallExtras {
    const int32_t *live_rows = nullptr;
    const unsigned long long *out_rows = nullptr;
    void *gu_out = nullptr;
};
CallExtras &call_extras();

// number of SMs of the current device (cached per device)
int sm_count();

// PMOE_PDL=0 in the environment disables programmatic dependent launch between the kernels of the
// split pipelines (they then run in plain stream order)
bool pdl_enabled();

// Default on: the split pipelines copy the routed rows of x into the workspace first and feed the
// gate/up GEMM with plain 2-D TMA tiles. PMOE_PREGATHER=0 switches to TMA gather4 straight from x
// (no pre-pass, smaller workspace, but gather4 issue rate then bounds the gate/up kernel).
bool pregather_enabled();

// How the split pipelines' gate/up GEMM gets the routed rows of x: PMOE_AGATHER=tma4 (0, TMA gather4),
// pre (1, row-gather pre-pass + plain tiles), lsu (2, cp.async gather by extra warps inside the kernel);
// unset = -1 = chosen per call: lsu for compute-bound calls of narrow layers on the one-CTA kernels, pre
// otherwise (measured best of each)
int a_operand_mode();

// PMOE_DOWN_BULK=0/1 forces the down kernels' epilogue (scattered vector reductions / bulk reductions from a
// staging tile); unset = -1 = chosen per problem
int down_bulk_reduce_mode();

// PMOE_L2_AHEAD=n: the GEMM producers prefetch weight tiles n k-steps ahead of the ring into L2
int l2_prefetch_distance();

// PMOE_SHORT_A=0 switches off the short TMA boxes (row blocks with few routed rows move only those rows of the
// A operand and of the activation tile); read on every call so that tests can compare both settings
int short_boxes_mode();

// bpc = 2 runs the half-empty last pair of an expert as a single block on the one-CTA kernels (PMOE_PAIR_TAILS=0:
// as a pair, like every other one)
bool pair_tails_enabled();

// PMOE_DUAL=0/1 forces one / two row blocks per tile in the one-CTA bf16 gate/up kernel; unset = -1 = by size
int dual_blocks_mode();   // bit 0: loads, bit 1: activation stores

// which launches of a split pipeline run (pmoe_debug_set_phase_mask): 1 gather, 2 gate/up, 4 down; 8 = without the
// single-block tail launches of the bpc = 2 pipeline (to time the CTA-pair kernels alone)
int phase_mask();

}  // namespace pmoe
