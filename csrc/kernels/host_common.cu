// host_common.cu - status words, tensor-map encoding, device properties.
#include "host_common.h"
#include "sm100.cuh"

#include <cudaTypedefs.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

namespace cai {

static thread_local char g_err[512] = "";

const char* last_error() { return g_err; }
void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int current_device() {
    int d = 0;
    cudaGetDevice(&d);
    return d;
}

static constexpr int kMaxDev = 64;
static int* g_status[kMaxDev];
static int g_sms[kMaxDev];
static std::mutex g_mu;

int* status_words(int device) {
    if (device < 0 || device >= kMaxDev) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_status[device]) {
        int* p = nullptr;
        if (cudaMalloc(&p, 64 * sizeof(int)) != cudaSuccess) return nullptr;
        cudaMemset(p, 0, 64 * sizeof(int));
        g_status[device] = p;
    }
    return g_status[device];
}

int sm_count(int device) {
    if (device < 0 || device >= kMaxDev) return 0;
    if (!g_sms[device]) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
        g_sms[device] = n;
    }
    return g_sms[device];
}

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    });
    return fn;
}

static CUtensorMapDataType dtype_of(int elem_bytes) {
    switch (elem_bytes) {
        case 1: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
        case 2: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        default: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    }
}

bool encode_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                    uint32_t box_cols, uint32_t box_rows, int elem_bytes, bool swizzle128) {
    auto fn = encode_fn();
    if (!fn) {
        set_last_error("cuTensorMapEncodeTiled entry point unavailable");
        return false;
    }
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstr[1] = {ld * static_cast<uint64_t>(elem_bytes)};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, dtype_of(elem_bytes), 2, const_cast<void*>(base), gdim, gstr, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled(2d) failed: %d (base=%p rows=%llu cols=%llu ld=%llu box=%ux%u)",
                       (int)r, base, (unsigned long long)rows, (unsigned long long)cols,
                       (unsigned long long)ld, box_cols, box_rows);
        return false;
    }
    return true;
}

bool encode_tmap_3d(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t batch,
                    uint64_t ld_row, uint64_t ld_batch, uint32_t box_cols, uint32_t box_rows,
                    int elem_bytes) {
    auto fn = encode_fn();
    if (!fn) {
        set_last_error("cuTensorMapEncodeTiled entry point unavailable");
        return false;
    }
    cuuint64_t gdim[3] = {cols, rows, batch};
    cuuint64_t gstr[2] = {ld_row * static_cast<uint64_t>(elem_bytes),
                          ld_batch * static_cast<uint64_t>(elem_bytes)};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, dtype_of(elem_bytes), 3, const_cast<void*>(base), gdim, gstr, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled(3d) failed: %d", (int)r);
        return false;
    }
    return true;
}

}  // namespace cai

// ---- exported status API -------------------------------------------------------------
// Reads the first status word of the current device (0 = no kernel has given up on a wait)
// and optionally clears it. Synchronises the device.
CAI_API int cai_status_read(int clear) {
    int dev = cai::current_device();
    int* p = cai::status_words(dev);
    if (!p) return cai::CAI_K_CUDA;
    int v = 0;
    if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return cai::CAI_K_CUDA;
    if (clear && v) cudaMemset(p, 0, sizeof(int));
    return v;
}

// Time limit, in microseconds, of every wait of a kernel on a flag that another GPU sets (0 restores the
// default of about two seconds). Takes effect for kernels launched after the call returns.
CAI_API int cai_set_wait_limit_us(unsigned int us) {
    int* p = cai::status_words(cai::current_device());
    if (!p) return cai::CAI_K_CUDA;
    return cudaMemcpy(p + cai::kStatusWordLimitUs, &us, sizeof us, cudaMemcpyHostToDevice) == cudaSuccess ? 0 : cai::CAI_K_CUDA;
}

// Makes every kernel of the current device that sits in a bounded wait give up now: the status word is set
// to CAI_DEV_ABORTED_BY_HOST on a stream of its own, next to whatever is running (a watchdog calls this when a
// step overruns its deadline, so that the step unwinds instead of running out one wait limit per kernel).
CAI_API int cai_status_abort() {
    int* p = cai::status_words(cai::current_device());
    if (!p) return cai::CAI_K_CUDA;
    static thread_local cudaStream_t side = nullptr;
    if (!side && cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking) != cudaSuccess) return cai::CAI_K_CUDA;
    static const int code = cai::CAI_DEV_ABORTED_BY_HOST;
    if (cudaMemcpyAsync(p, &code, sizeof code, cudaMemcpyHostToDevice, side) != cudaSuccess) return cai::CAI_K_CUDA;
    return cudaStreamSynchronize(side) == cudaSuccess ? 0 : cai::CAI_K_CUDA;
}

CAI_API const char* cai_last_error() { return cai::last_error(); }

CAI_API int cai_sm_count() { return cai::sm_count(cai::current_device()); }
