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
    const int R = (H + kNormWarpCols - 1) / kNormWarpCols;
    const int parts = rows < CAI_RMSNORM_STATIC_PARTS ? rows : CAI_RMSNORM_STATIC_PARTS;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // every CTA writes its whole row of the scratch before the reduction reads rows [0, parts)
    rmsnorm_bwd_kernel<<<parts, kNormThreads, H * sizeof(float), st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(g), rstd,
        static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), scratch, rows, H, dx_accumulate, R);
    if (cudaGetLastError() != cudaSuccess) {
        set_last_error("rmsnorm_bwd_static: launch failed");
        return CAI_K_CUDA;
    }
    reduce_parts_kernel<<<(H + 31) / 32, 256, 0, st>>>(scratch, dg, parts, H, dg_accumulate);
    if (cudaGetLastError() != cudaSuccess) {
        set_last_error("rmsnorm_bwd_static: reduction launch failed");
        return CAI_K_CUDA;
    }
    return CAI_K_OK;
}
