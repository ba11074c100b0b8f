// ipc.cu - peer mapping of arenas between the ranks of one box.
//
// Each rank exports the allocation that holds its arena as a CUDA IPC handle (plus the offset of
// the arena inside that allocation); every other rank of the box opens it, which maps the peer's
// arena into its own address space and enables NVLink peer access. The fused kernels then address
// any tensor of any member as base[member] + arena offset. Replaces the reference's NVSHMEM
// symmetric heap (src/cuda/cai_nvshmem.cu:16-50), which is not installed here.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <string.h>

#include "../kernels/host_common.h"
#include "../runtime/cai_runtime.h"

using namespace cai;

// Writes a 64-byte IPC handle and the offset of `ptr` inside its allocation.
CAI_API int cai_ipc_export(void* ptr, void* handle64, unsigned long long* offset) {
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) {
        set_last_error("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(cudaGetLastError()));
        return CAI_K_CUDA;
    }
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    CUdeviceptr base = 0;
    size_t size = 0;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn ||
        reinterpret_cast<PFN_cuMemGetAddressRange_v3020>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) {
        set_last_error("cuMemGetAddressRange failed");
        return CAI_K_CUDA;
    }
    *offset = reinterpret_cast<CUdeviceptr>(ptr) - base;
    return 0;
}

// Maps a peer's allocation and returns the address that corresponds to the exported pointer.
CAI_API int cai_ipc_open(const void* handle64, unsigned long long offset, void** out) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* base = nullptr;
    if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        set_last_error("cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(cudaGetLastError()));
        return CAI_K_CUDA;
    }
    *out = static_cast<uint8_t*>(base) + offset;
    return 0;
}

CAI_API int cai_ipc_close(void* mapped, unsigned long long offset) {
    return cudaIpcCloseMemHandle(static_cast<uint8_t*>(mapped) - offset) == cudaSuccess ? 0 : CAI_K_CUDA;
}
