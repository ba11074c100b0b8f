// tcgen05_probe.cu - cycle counts that decide how a tcgen05 kernel has to be laid out on a B200.
//
// One CTA (or one per SM) runs three experiments on operands that are all zeros in shared memory:
//   mma      cycles per tcgen05.mma for the operand forms the GEMM and attention kernels use, issued back to back
//            by one thread (the tensor pipe's rate for that form);
//   handoff  the round trip "issuing thread commits -> N warps wait, arrive -> issuing thread waits", with and
//            without MMAs in front of the commit (what a softmax step between two MMA groups costs at least);
//   wait     what an mbarrier wait that is ALREADY satisfied costs the issuing thread between two groups of MMAs
//            (the tensor pipe idles for most of it: the thread runs at most about one MMA ahead).
// Every wait is bounded; the kernels use no global memory besides the result words. Usage: tcgen05_probe [mma|handoff|wait]
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../kernels/sm100.cuh"

using namespace cai;

namespace {

constexpr int kOperandBytes = 98304;  // A: 32 KiB (128 rows x 128 bf16), B: 64 KiB (256 rows x 128 bf16)
constexpr int kSmemBytes = kOperandBytes + 1024 + 256;

struct Smem {
    uint8_t* a;
    uint8_t* b;
    uint64_t* bar;
    uint32_t* slot;
    volatile int* abort_flag;
};

__device__ Smem carve_and_clear(uint8_t* raw, int nbars) {
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    Smem m;
    m.a = smem;
    m.b = smem + 32768;
    m.bar = reinterpret_cast<uint64_t*>(smem + kOperandBytes);
    m.slot = reinterpret_cast<uint32_t*>(m.bar + 16);
    m.abort_flag = reinterpret_cast<volatile int*>(m.slot + 1);
    for (int i = threadIdx.x; i < kOperandBytes / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
    if (threadIdx.x == 0) {
        for (int i = 0; i < nbars; ++i) mbar_init(&m.bar[i], 1);
        *m.abort_flag = 0;
        mbar_fence_init();
    }
    fence_proxy_async_smem();
    if (threadIdx.x < 32) {
        tmem_alloc(m.slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    return m;
}

__device__ void release_tmem(uint32_t tmem_base) {
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- mma: FORM 0..2 = both operands K-major in shared memory, N = 256 / 128 / 64; 3 = N = 64 alternating between two
// accumulators (S and dP of an attention half step); 4 = A from tensor memory, B MN-major, N = 128 (P V, dS K).
template <int FORM>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int groups, long long* out) {
    extern __shared__ uint8_t raw[];
    const Smem m = carve_and_clear(raw, 1);
    const uint32_t tb = *m.slot;
    if (threadIdx.x == 0) {
        const uint64_t da = umma_smem_desc_sw128(smem_u32(m.a), 0, 1024), db = umma_smem_desc_sw128(smem_u32(m.b), 0, 1024);
        const uint64_t db_mn = umma_smem_desc_sw128(smem_u32(m.b), 16384, 1024);
        constexpr int N = FORM == 0 ? 256 : (FORM == 1 || FORM == 4) ? 128 : 64;
        constexpr uint32_t idesc = umma_idesc_bf16(128, N, 0, FORM == 4 ? 1 : 0);
        constexpr uint32_t bsub = N * 128;  // bytes of one 64-column sub-tile of a K-major B
        const long long t0 = clock64();
        for (int g = 0; g < groups; ++g) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t a_off = ((k >> 2) * 16384 + (k & 3) * 32) >> 4, b_off = ((k >> 2) * bsub + (k & 3) * 32) >> 4;
                if (FORM == 4) umma_f16_ts(tb, tb + 256 + k * 8, db_mn + ((k * 2048) >> 4), idesc, k > 0);
                else umma_f16_ss(tb + (FORM == 3 ? (k & 1) * 64 : 0), da + a_off, db + b_off, idesc, k > 1);
            }
        }
        umma_commit(&m.bar[0]);
        const bool ok = mbar_wait(&m.bar[0], 0, m.abort_flag, nullptr, 0);
        out[blockIdx.x] = ok ? clock64() - t0 : -1;
    }
    release_tmem(tb);
}

// ---- handoff: thread 0 issues `mmas` MMAs (N = 128), commits to bar 0; `nwarps` warps wait on it and arrive (one
// arrival per warp) on bar 1; thread 0 waits for that.
__global__ void __launch_bounds__(640, 1) handoff_kernel(int rounds, int nwarps, int mmas, long long* out) {
    extern __shared__ uint8_t raw[];
    const Smem m = carve_and_clear(raw, 1);
    if (threadIdx.x == 0) {
        mbar_init(&m.bar[1], nwarps);
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t tb = *m.slot;
    const int warp = threadIdx.x >> 5;
    bool ok = true;
    if (threadIdx.x == 0) {
        const uint64_t da = umma_smem_desc_sw128(smem_u32(m.a), 0, 1024), db = umma_smem_desc_sw128(smem_u32(m.b), 0, 1024);
        constexpr uint32_t idesc = umma_idesc_bf16(128, 128, 0, 0);
        const long long t0 = clock64();
        for (int i = 0; i < rounds && ok; ++i) {
            if (mmas) {
                for (int k = 0; k < mmas; ++k) umma_f16_ss(tb, da + 2 * (k & 3), db + 2 * (k & 3), idesc, 1);
                umma_commit(&m.bar[0]);
            } else {
                mbar_arrive(&m.bar[0]);
            }
            ok = mbar_wait(&m.bar[1], i & 1, m.abort_flag, nullptr, 0);
            tc_fence_after();
        }
        out[0] = ok ? clock64() - t0 : -1;
    } else if (warp >= 4 && warp < 4 + nwarps) {
        for (int i = 0; i < rounds && ok; ++i) {
            ok = mbar_wait_warp(&m.bar[0], i & 1, m.abort_flag, nullptr, 0);
            tc_fence_after();
            tc_fence_before();
            mbar_arrive_warp(&m.bar[1]);
        }
    }
    release_tmem(tb);
}

// ---- wait: per step, `nwaits` waits on barriers whose phase has long completed, then 4 MMAs with N = 256 (512 cycles of
// tensor work) and a commit. STYLE 0: the bounded wait loop the kernels use; 1: a single mbarrier.try_wait.
template <int STYLE>
__global__ void __launch_bounds__(128, 1) satisfied_wait_kernel(int steps, int nwaits, long long* out) {
    extern __shared__ uint8_t raw[];
    const Smem m = carve_and_clear(raw, 8);  // bars 1-4 are never arrived on: their parity-1 phase reads as complete
    const uint32_t tb = *m.slot;
    if (threadIdx.x == 0) {
        const uint64_t da = umma_smem_desc_sw128(smem_u32(m.a), 0, 1024), db = umma_smem_desc_sw128(smem_u32(m.b), 0, 1024);
        constexpr uint32_t idesc = umma_idesc_bf16(128, 256, 0, 0);
        bool ok = true;
        const long long t0 = clock64();
        for (int s = 0; s < steps && ok; ++s) {
            for (int w = 0; w < nwaits && ok; ++w) {
                if (STYLE == 0) ok = mbar_wait(&m.bar[1 + (w & 3)], 1, m.abort_flag, nullptr, 0);
                else ok = mbar_try_wait(&m.bar[1 + (w & 3)], 1);
                tc_fence_after();
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_f16_ss(tb, da + 2 * k, db + 2 * k, idesc, 1);
            umma_commit(&m.bar[5 + (s & 1)]);  // like freeing a stage; nobody waits on it here
        }
        umma_commit(&m.bar[0]);
        const bool fin = mbar_wait(&m.bar[0], 0, m.abort_flag, nullptr, 0);
        out[0] = (ok && fin) ? clock64() - t0 : -1;
    }
    release_tmem(tb);
}

template <typename K>
void prepare(K kernel) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
        std::fprintf(stderr, "cudaFuncSetAttribute failed\n");
        std::exit(1);
    }
}

void sync_or_die() {
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        std::fprintf(stderr, "kernel failed: %s\n", cudaGetErrorString(e));
        std::exit(1);
    }
}

template <int FORM>
void run_mma(const char* name, long long* out) {
    const int groups = 512;
    prepare(mma_rate_kernel<FORM>);
    for (int grid : {1, 148}) {
        for (int rep = 0; rep < 2; ++rep) {
            mma_rate_kernel<FORM><<<grid, 128, kSmemBytes>>>(groups, out);
            sync_or_die();
        }
        long long h[148];
        cudaMemcpy(h, out, grid * sizeof(long long), cudaMemcpyDeviceToHost);
        long long mx = 0;
        for (int b = 0; b < grid; ++b) mx = h[b] > mx ? h[b] : mx;
        std::printf("mma      %-46s CTAs %3d  cycles per MMA %6.1f\n", name, grid, static_cast<double>(mx) / (groups * 8.0));
    }
}

}  // namespace

int main(int argc, char** argv) {
    const char* what = argc > 1 ? argv[1] : "all";
    const bool all = !std::strcmp(what, "all");
    long long* out = nullptr;
    if (cudaMalloc(&out, 256 * sizeof(long long)) != cudaSuccess) {
        std::fprintf(stderr, "no CUDA device\n");
        return 1;
    }
    if (all || !std::strcmp(what, "mma")) {
        run_mma<0>("smem x smem, K-major, N = 256 (ideal 128)", out);
        run_mma<1>("smem x smem, K-major, N = 128 (ideal 64)", out);
        run_mma<2>("smem x smem, K-major, N = 64 (ideal 32)", out);
        run_mma<3>("smem x smem, N = 64, two accumulators in turn", out);
        run_mma<4>("tmem x smem (MN-major B), N = 128 (ideal 64)", out);
    }
    if (all || !std::strcmp(what, "handoff")) {
        prepare(handoff_kernel);
        const int rounds = 2000;
        for (int mmas : {0, 1, 4, 8})
            for (int nwarps : {1, 16}) {
                for (int rep = 0; rep < 2; ++rep) {
                    handoff_kernel<<<1, 640, kSmemBytes>>>(rounds, nwarps, mmas, out);
                    sync_or_die();
                }
                long long h;
                cudaMemcpy(&h, out, sizeof(h), cudaMemcpyDeviceToHost);
                std::printf("handoff  %d MMAs (N = 128, %3d cycles of math) + commit, %2d waiting warps: round trip %6.1f cycles\n", mmas,
                            mmas * 64, nwarps, static_cast<double>(h) / rounds);
            }
    }
    if (all || !std::strcmp(what, "wait")) {
        prepare(satisfied_wait_kernel<0>);
        prepare(satisfied_wait_kernel<1>);
        const int steps = 1024;
        for (int style = 0; style < 2; ++style)
            for (int nwaits : {0, 1, 2, 4}) {
                for (int rep = 0; rep < 2; ++rep) {
                    if (style == 0) satisfied_wait_kernel<0><<<1, 128, kSmemBytes>>>(steps, nwaits, out);
                    else satisfied_wait_kernel<1><<<1, 128, kSmemBytes>>>(steps, nwaits, out);
                    sync_or_die();
                }
                long long h;
                cudaMemcpy(&h, out, sizeof(h), cudaMemcpyDeviceToHost);
                std::printf("wait     %-22s %d satisfied waits + 4 MMAs (512 cycles of math) per step: %6.1f cycles per step\n",
                            style == 0 ? "bounded wait loop," : "single try_wait,", nwaits, static_cast<double>(h) / steps);
            }
    }
    cudaFree(out);
    return 0;
}
