// Implementation of the allocation-free entry point declared in ../lme_noalloc.h.
#include "common.cuh"
#include "../lme_api.h"
#include "../lme_noalloc.h"

namespace lme {

// Workspace for the weight-gradient partial sums.  In host code this name is only a handle for the runtime's symbol
// table, never a device pointer: the address a kernel can use is obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_scratch[LME_STATIC_SCRATCH_FLOATS];

static constexpr int kMaxDevices = 64;
static float* g_static_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the workspace on the current device (resolved once per device).
static int static_scratch_address(float** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return LME_ERR_LAUNCH;
    if (g_static_scratch_addr[dev] == nullptr) {
        float* p = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch) != cudaSuccess || p == nullptr)
            return LME_ERR_LAUNCH;
        g_static_scratch_addr[dev] = p;
    }
    *out = g_static_scratch_addr[dev];
    return LME_OK;
}

}  // namespace lme

extern "C" int lme_rmsnorm_bwd_static_scratch(const void* dy, const void* h, const void* w, const float* rstd,
                                              const void* dres, void* dx, float* dw, int dw_accumulate, int T, int H,
                                              void* stream) {
    if (T < 0 || H <= 0) return LME_ERR_SHAPE;
    const long long need = static_cast<long long>(lme_rmsnorm_bwd_partial_rows(T)) * H;
    if (need > LME_STATIC_SCRATCH_FLOATS) return LME_ERR_TOO_LARGE;
    float* scratch = nullptr;
    int rc = lme::static_scratch_address(&scratch);
    if (rc != LME_OK) return rc;
    return lme_rmsnorm_bwd(dy, h, w, rstd, dres, dx, scratch, dw, dw_accumulate, T, H, stream);
}
