// placeholder until the mxfp8 kernels land
#include "host_common.h"
namespace pmoe {
__device__ int g_status_mxfp8 = 0;
int status_fetch_mxfp8(int *value, bool reset) {
    if (value) PMOE_CUDA_OK(cudaMemcpyFromSymbol(value, g_status_mxfp8, sizeof(int)));
    if (reset) {
        const int zero = 0;
        PMOE_CUDA_OK(cudaMemcpyToSymbol(g_status_mxfp8, &zero, sizeof(int)));
    }
    return PMOE_OK;
}
}
extern "C" size_t pmoe_fused_moe_mxfp8_workspace_bytes(int, int, int, int, int) { return 0; }
extern "C" int pmoe_fused_moe_mxfp8_ws(const void *, const void *, const void *, const void *, const void *, const void *, void *, const int32_t *, const int32_t *, const int32_t *, const float *, int, int, int, int, int, int, int, int, int, int, int, int, void *, size_t, pmoe_stream_t) {
    return pmoe::set_error(PMOE_ERR_UNSUPPORTED, "mxfp8 not built yet");
}
extern "C" int pmoe_fused_moe_mxfp8(const void *, const void *, const void *, const void *, const void *, const void *, void *, const int32_t *, const int32_t *, const int32_t *, const float *, int, int, int, int, int, int, int, int, int, int, int, int, pmoe_stream_t) {
    return pmoe::set_error(PMOE_ERR_UNSUPPORTED, "mxfp8 not built yet");
}
