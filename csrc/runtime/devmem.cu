// devmem.cu - the handful of CUDA runtime calls a host program needs to drive the executor without
// linking CUDA itself: pick a device, allocate the arena, move bytes. The GPU-free host library
// (libcai_host.so) reaches these through dlopen when its device backend is selected, which is how
// one `cai_init` serves both the analytic and the real backend (the reference's cai_init tries its
// CUDA backend first and falls back to the analytic one, src/runtime.c:32-73).
#include <cuda_runtime.h>

#include "../kernels/host_common.h"
#include "cai_runtime.h"

using namespace cai;

CAI_API int cai_dev_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

CAI_API int cai_dev_set(int device) {
    if (cudaSetDevice(device) != cudaSuccess) {
        set_last_error("cudaSetDevice(%d): %s", device, cudaGetErrorString(cudaGetLastError()));
        return CAI_K_CUDA;
    }
    return 0;
}

CAI_API int cai_dev_malloc(void** out, unsigned long long nbytes) {
    if (cudaMalloc(out, nbytes) != cudaSuccess) {
        set_last_error("cudaMalloc(%llu bytes): %s", nbytes, cudaGetErrorString(cudaGetLastError()));
        return CAI_K_CUDA;
    }
    return 0;
}

CAI_API int cai_dev_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : CAI_K_CUDA; }

CAI_API int cai_dev_memset(void* p, int value, unsigned long long nbytes) {
    return cudaMemset(p, value, nbytes) == cudaSuccess ? 0 : CAI_K_CUDA;
}

// Blocking copies (set-up, parameter initialisation, the per-step loss): the step itself never waits on them.
CAI_API int cai_dev_h2d(void* dst, const void* src, unsigned long long nbytes) {
    return cudaMemcpy(dst, src, nbytes, cudaMemcpyHostToDevice) == cudaSuccess ? 0 : CAI_K_CUDA;
}
CAI_API int cai_dev_d2h(void* dst, const void* src, unsigned long long nbytes) {
    return cudaMemcpy(dst, src, nbytes, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : CAI_K_CUDA;
}

// Stream-ordered host->device copy on one of the executor's streams (the batch of the next step).
CAI_API int cai_dev_h2d_async(void* dst, const void* src, unsigned long long nbytes, void* stream) {
    return cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : CAI_K_CUDA;
}

CAI_API int cai_dev_host_alloc(void** out, unsigned long long nbytes) {
    return cudaMallocHost(out, nbytes) == cudaSuccess ? 0 : CAI_K_CUDA;
}
CAI_API int cai_dev_host_free(void* p) { return cudaFreeHost(p) == cudaSuccess ? 0 : CAI_K_CUDA; }
