// gemm_fp8_blockscaled.cu - fp8 (e4m3) GEMM with 1x128 / 128x128 block scales on tcgen05.
//
//   C[M,N] = sum over k-blocks kb of  sa[m, kb] * sb[n / 128, kb] * (Aq[m, kb-block] . Bq[n, kb-block])
//
// Aq [M,K] and Bq [N,K] are e4m3, K-major; sa [M, K/128] holds one fp32 scale per row and 128-wide
// k-block (activations), sb [ceil(N/128), K/128] one per 128x128 block (weights). These are not the
// scales the tensor core applies by itself (that format is 32-element UE8M0), so every k-block is
// its own MMA group: the MMA warp issues the four K=32 tcgen05.mma (kind::f8f6f4) of a 128-deep
// block into one of two TMEM buffers, eight epilogue warps read that fp32 partial back with
// tcgen05.ld, scale it and add it to accumulators kept in registers while the tensor core works on
// the next block in the other buffer. TMA (128-byte swizzle, one 128-byte row = 128 k-elements)
// feeds a 4-stage shared-memory ring. Persistent, one CTA per SM, 128x256 tiles.
//
// The reference only names the dtype (`param_dtype fp8e4m3`, include/cai_tensor.h:14-22) and has no
// fp8 arithmetic anywhere.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "cai_kernels.h"
#include "host_common.h"
#include "norm_kernels.cuh"
#include "sm100.cuh"

namespace cai {

namespace f8 {
constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 128;   // e4m3 elements = bytes per row of a stage
constexpr int kUmmaK = 32;
constexpr int kStages = 4;
constexpr int kAStage = kBM * kBK;
constexpr int kBStage = kBN * kBK;
constexpr int kStage = kAStage + kBStage;
constexpr int kThreads = 320;  // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue
constexpr int kSmem = kStages * kStage + 1024 + 256;
}  // namespace f8

struct GemmFp8Params {
    int M, N, K;
    const float* sa;   // [M, K/128]
    const float* sb;   // [ceil(N/128), K/128]
    void* C;
    const void* R;
    long long ldc, ldr;
    int epi;
    int tiles_m, tiles_n;
    int* status;
};

// kind::f8f6f4, A = B = e4m3 (format 0), D = f32, both K-major
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ void umma_f8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(f8::kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmFp8Params p) {
    using namespace f8;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + kStages * kAStage;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStage);
    uint64_t* full = bars;
    uint64_t* empty = bars + kStages;
    uint64_t* part_full = bars + 2 * kStages;        // [2] a k-block's partial product is in TMEM
    uint64_t* part_empty = bars + 2 * kStages + 2;   // [2] the epilogue warps have read it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&part_full[a], 1);
            mbar_init(&part_empty[a], 8);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * kBN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int num_kb = p.K / kBK;
    const int cta = blockIdx.x, ncta = gridDim.x;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = cta; tile < num_tiles && ok; tile += ncta) {
                const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_TMA_EMPTY)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[s], kStage);
                    tma_load_2d(sA + s * kAStage, &tmA, &full[s], kb * kBK, tm * kBM);
                    tma_load_2d(sB + s * kBStage, &tmB, &full[s], kb * kBK, tn * kBN);
                    if (++s == kStages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
            if (!ok)
                for (int i = 0; i < 32; ++i) __nanosleep(50000);  // let copies in flight land before the CTA's memory goes
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_e4m3(kBM, kBN);
            int s = 0;
            uint32_t ph = 0;
            uint32_t it = 0;  // k-blocks issued by this CTA: TMEM buffer = it & 1
            bool ok = true;
            for (int tile = cta; tile < num_tiles && ok; tile += ncta) {
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t buf = it & 1;
                    if (!mbar_wait(&part_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_TMEM_EMPTY) ||
                        !mbar_wait(&full[s], ph, abort_flag, p.status, CAI_DEV_TIMEOUT_TMA_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(sA + s * kAStage), b_base = smem_u32(sB + s * kBStage);
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k)
                        umma_f8_ss(tmem_base + buf * kBN, umma_smem_desc_sw128(a_base + k * kUmmaK, 0, 1024),
                                   umma_smem_desc_sw128(b_base + k * kUmmaK, 0, 1024), idesc, k != 0 ? 1u : 0u);
                    umma_commit(&empty[s]);
                    umma_commit(&part_full[buf]);
                    if (++s == kStages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else {
        // ---------------- epilogue warps: scale-and-add every k-block, then write the tile
        const int q = warp & 3;           // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2; // which 128 columns of the tile
        uint32_t it = 0;
        bool ok = true;
        for (int tile = cta; tile < num_tiles && ok; tile += ncta) {
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            const long long row = static_cast<long long>(tm) * kBM + q * 32 + lane;
            const int col0 = tn * kBN + half * 128;
            const bool row_ok = row < p.M;
            const bool cols_ok = col0 < p.N;
            const float* sa_row = p.sa + (row_ok ? row : 0) * num_kb;
            const float* sb_row = p.sb + static_cast<long long>(cols_ok ? col0 / 128 : 0) * num_kb;
            float acc[128];
#pragma unroll
            for (int e = 0; e < 128; ++e) acc[e] = 0.f;
            float s_next = sa_row[0] * sb_row[0];
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const uint32_t buf = it & 1;
                const float s = s_next;
                if (kb + 1 < num_kb) s_next = sa_row[kb + 1] * sb_row[kb + 1];
                if (!mbar_wait(&part_full[buf], (it >> 1) & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_TMEM_FULL)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kBN + half * 128;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[c * 32 + e] = fmaf(s, __uint_as_float(r[e]), acc[c * 32 + e]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&part_empty[buf]);
            }
            if (!ok || !row_ok || !cols_ok) continue;
            if (p.epi == CAI_EPI_F32) {
                float* crow = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (col0 + j * 4 >= p.N) break;
                    *reinterpret_cast<float4*>(crow + j * 4) = make_float4(acc[j * 4], acc[j * 4 + 1], acc[j * 4 + 2], acc[j * 4 + 3]);
                }
            } else {
                __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
                const __nv_bfloat16* rrow =
                    p.epi == CAI_EPI_BF16_RESIDUAL ? reinterpret_cast<const __nv_bfloat16*>(p.R) + row * p.ldr + col0 : nullptr;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (col0 + j * 8 >= p.N) break;
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = acc[j * 8 + e];
                    if (rrow) {
                        float rf[8];
                        unpack8(*reinterpret_cast<const uint4*>(rrow + j * 8), rf);
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] += rf[e];
                    }
                    *reinterpret_cast<uint4*>(crow + j * 8) = pack8(v);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 2 * f8::kBN);
}

// ------------------------------------------------------------------ quantisation
// One warp per (row, 128-column block): amax -> scale = amax / 448, q = x / scale.
__global__ void __launch_bounds__(256)
quant_rows_1x128_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_fp8_storage_t* __restrict__ q, long long ldq,
                        float* __restrict__ scale, int rows, int cols) {
    const int kb_n = cols / 128;
    const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= static_cast<long long>(rows) * kb_n) return;
    const long long r = w / kb_n;
    const int kb = static_cast<int>(w % kb_n);
    const uint2 raw = *reinterpret_cast<const uint2*>(x + r * ldx + kb * 128 + lane * 4);
    float v[4] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y)};
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = warp_max(amax);
    const float s = amax > 0.f ? amax / 448.f : 1.f;
    const float inv = 1.f / s;
    uint32_t out = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e)
        out |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[e] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * e);
    *reinterpret_cast<uint32_t*>(q + r * ldq + kb * 128 + lane * 4) = out;
    if (lane == 0) scale[r * kb_n + kb] = s;
}

// One CTA per 128x128 block of a weight [rows, cols]: a common scale; optionally also writes the
// transposed quantised block (qt [cols, rows], for the input-gradient GEMM that contracts over rows).
__global__ void __launch_bounds__(256)
quant_blocks_128x128_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, __nv_fp8_storage_t* __restrict__ q, long long ldq,
                            __nv_fp8_storage_t* __restrict__ qt, long long ldqt, float* __restrict__ scale,
                            float* __restrict__ scale_t, int rows, int cols) {
    __shared__ __nv_bfloat16 tile[128][130];
    __shared__ float red[8];
    const int bc = blockIdx.x, br = blockIdx.y;
    const int nbc = gridDim.x, nbr = gridDim.y;
    float amax = 0.f;
    for (int i = threadIdx.x; i < 128 * 128; i += 256) {
        const int r = i >> 7, c = i & 127;
        const long long gr = static_cast<long long>(br) * 128 + r;
        const int gc = bc * 128 + c;
        const float v = (gr < rows && gc < cols) ? __bfloat162float(w[gr * ldw + gc]) : 0.f;
        tile[r][c] = __float2bfloat16(v);
        amax = fmaxf(amax, fabsf(v));
    }
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) amax = fmaxf(amax, red[k]);
    const float s = amax > 0.f ? amax / 448.f : 1.f;
    const float inv = 1.f / s;
    if (threadIdx.x == 0) {
        scale[static_cast<long long>(br) * nbc + bc] = s;
        if (scale_t) scale_t[static_cast<long long>(bc) * nbr + br] = s;
    }
    for (int i = threadIdx.x; i < 128 * 128; i += 256) {
        const int r = i >> 7, c = i & 127;
        const long long gr = static_cast<long long>(br) * 128 + r;
        const int gc = bc * 128 + c;
        if (gr < rows && gc < cols) q[gr * ldq + gc] = __nv_cvt_float_to_fp8(__bfloat162float(tile[r][c]) * inv, __NV_SATFINITE, __NV_E4M3);
    }
    if (qt)
        for (int i = threadIdx.x; i < 128 * 128; i += 256) {
            const int c = i >> 7, r = i & 127;   // consecutive threads walk a column of the block = a row of qt
            const long long gr = static_cast<long long>(br) * 128 + r;
            const int gc = bc * 128 + c;
            if (gr < rows && gc < cols)
                qt[static_cast<long long>(gc) * ldqt + gr] = __nv_cvt_float_to_fp8(__bfloat162float(tile[r][c]) * inv, __NV_SATFINITE, __NV_E4M3);
        }
}

}  // namespace cai

using namespace cai;

CAI_API int cai_gemm_fp8_blockscaled(const void* Aq, const float* sa, const void* Bq, const float* sb, void* C, const void* R,
                                     int M, int N, int K, long long lda, long long ldb, long long ldc, long long ldr, int epi,
                                     void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return CAI_K_OK;
    if ((K % 128) || (lda & 15) || (ldb & 15) || (N & 7) || (epi != CAI_EPI_BF16 && epi != CAI_EPI_F32 && epi != CAI_EPI_BF16_RESIDUAL) ||
        (epi != CAI_EPI_F32 && (ldc & 7)) || (epi == CAI_EPI_F32 && (ldc & 3)) || (epi == CAI_EPI_BF16_RESIDUAL && (!R || (ldr & 7)))) {
        set_last_error("gemm_fp8: K %% 128, lda/ldb %% 16, N %% 8 and an aligned C are required (M=%d N=%d K=%d)", M, N, K);
        return CAI_K_BAD_ARG;
    }
    const int dev = current_device();
    CUtensorMap tmA, tmB;
    if (!encode_tmap_2d(&tmA, Aq, M, K, lda, f8::kBK, f8::kBM, 1) || !encode_tmap_2d(&tmB, Bq, N, K, ldb, f8::kBK, f8::kBN, 1))
        return CAI_K_BAD_ARG;
    static bool configured[64] = {};
    if (!configured[dev & 63]) {
        if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, f8::kSmem) != cudaSuccess) {
            set_last_error("cudaFuncSetAttribute(gemm_fp8) failed");
            return CAI_K_CUDA;
        }
        configured[dev & 63] = true;
    }
    GemmFp8Params p;
    p.M = M; p.N = N; p.K = K;
    p.sa = sa; p.sb = sb;
    p.C = C; p.R = R; p.ldc = ldc; p.ldr = ldr; p.epi = epi;
    p.tiles_m = (M + f8::kBM - 1) / f8::kBM;
    p.tiles_n = (N + f8::kBN - 1) / f8::kBN;
    p.status = status_words(dev);
    const int tiles = p.tiles_m * p.tiles_n;
    const int sms = sm_count(dev);
    gemm_fp8_kernel<<<tiles < sms ? tiles : sms, f8::kThreads, f8::kSmem, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, p);
    if (cudaGetLastError() != cudaSuccess) {
        set_last_error("gemm_fp8 launch failed");
        return CAI_K_CUDA;
    }
    return CAI_K_OK;
}

CAI_API int cai_quant_rows_1x128(const void* x, long long ldx, void* q, long long ldq, float* scale, int rows, int cols,
                                 void* stream) {
    if (cols % 128 || (ldx & 3) || (ldq & 3)) {
        set_last_error("quant_rows: columns must be a multiple of 128");
        return CAI_K_BAD_ARG;
    }
    const long long warps = static_cast<long long>(rows) * (cols / 128);
    if (warps == 0) return CAI_K_OK;
    quant_rows_1x128_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<__nv_fp8_storage_t*>(q), ldq, scale, rows, cols);
    return cudaGetLastError() == cudaSuccess ? 0 : CAI_K_CUDA;
}

CAI_API int cai_quant_blocks_128x128(const void* w, long long ldw, void* q, long long ldq, void* qt, long long ldqt, float* scale,
                                     float* scale_t, int rows, int cols, void* stream) {
    if (rows <= 0 || cols <= 0) return CAI_K_OK;
    dim3 grid((cols + 127) / 128, (rows + 127) / 128);
    quant_blocks_128x128_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(w), ldw, static_cast<__nv_fp8_storage_t*>(q), ldq, static_cast<__nv_fp8_storage_t*>(qt),
        ldqt, scale, scale_t, rows, cols);
    return cudaGetLastError() == cudaSuccess ? 0 : CAI_K_CUDA;
}
