// rmsnorm_bwd_static.cu - the allocation-free variant of RMSNorm backward (see the header for who
// needs it and the rules that come with it). Same device code as cai_rmsnorm_bwd(); the scratch for
// the per-CTA partial gain gradients is a file-scope device array of fixed size.
#include "rmsnorm_bwd_static.h"

#include "host_common.h"
#include "norm_kernels.cuh"

namespace cai {

// Partial gain gradients, one row of H floats per CTA. Lives in the library image on every GPU
// that loads it. In host code this name is only a handle for the runtime, not a device address:
// the address is fetched per device with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_rmsnorm_static_scratch[CAI_RMSNORM_STATIC_PARTS * CAI_RMSNORM_STATIC_MAX_H];

constexpr int kStaticMaxDev = 64;
static float* g_scratch_addr[kStaticMaxDev];  // device address of the array, per device (0 = not looked up yet)

}  // namespace cai

using namespace cai;

CAI_API int cai_rmsnorm_bwd_static(const void* x, const void* g, const float* rstd, const void* dy, void* dx, float* dg,
                                   int rows, int H, int dx_accumulate, int dg_accumulate, void* stream) {
    if (rows <= 0) return CAI_K_OK;
    if (H <= 0 || (H & 7) || H > CAI_RMSNORM_STATIC_MAX_H) {
        set_last_error("rmsnorm_bwd_static: H=%d is not supported (multiple of 8, at most %d); use cai_rmsnorm_bwd with "
                       "a scratch buffer for larger rows", H, CAI_RMSNORM_STATIC_MAX_H);
        return CAI_K_BAD_ARG;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDev) {
        set_last_error("rmsnorm_bwd_static: no usable current device");
        return CAI_K_CUDA;
    }
    if (!g_scratch_addr[dev]) {
        // one-time set-up for this device (it is current): resolve the array's device address
        float* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_static_scratch);
        if (e != cudaSuccess || !p) {
            set_last_error("rmsnorm_bwd_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return CAI_K_CUDA;
        }
        g_scratch_addr[dev] = p;
    }
    float* scratch = g_scratch_addr[dev];
    // the gain-gradient kernel writes rows [0, parts) of the scratch in full before the reduction reads them
    if (launch_rmsnorm_bwd(x, g, rstd, dy, dx, dg, scratch, CAI_RMSNORM_STATIC_PARTS, sm_count(dev), rows, H, dx_accumulate,
                           dg_accumulate, static_cast<cudaStream_t>(stream)) != 0) {
        set_last_error("rmsnorm_bwd_static: launch failed");
        return CAI_K_CUDA;
    }
    return CAI_K_OK;
}
