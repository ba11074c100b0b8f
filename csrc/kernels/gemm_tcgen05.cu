// gemm_tcgen05.cu - persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] = alpha * sum_k A(m,k) * B(n,k)   (+ epilogue)
//
// One CTA per SM walks output tiles of 128 x BN (BN = 128 or 256). Warp 0 feeds a multi-stage
// shared-memory ring with TMA tiled loads (128-byte swizzle); warp 1 issues tcgen05.mma from one
// thread with the fp32 accumulator in tensor memory; warps 2-5 drain the accumulator with
// tcgen05.ld and run the epilogue. Two accumulators live in TMEM so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Either operand may be K-major (the reduction dimension is contiguous in memory) or MN-major
// (the M / N dimension is contiguous), which covers forward (X * W^T), input-gradient (dY * W) and
// weight-gradient (dY^T * X) products without materialising a transpose.
//
// Replaces the one-thread-per-output fp32 GEMMs of the reference
// (src/cuda/cai_gpu_train.cu:40-74) and folds its add_k / zero_k passes
// (src/cuda/cai_kernels.cu:161-164, cai_gpu_train.cu:75-78) into the epilogue.
#include "cai_kernels.h"
#include "host_common.h"
#include "sm100.cuh"

namespace cai {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kUmmaK = 16;
constexpr int kAStageBytes = kBM * kBK * 2;
constexpr int kGemmThreads = 192;

struct GemmParams {
    int M, N, K;
    int a_mn, b_mn;
    int epi;
    float alpha;
    void* C;
    const void* R;
    long long ldc, ldr;
    int tiles_m, tiles_n, group_m;
    int* status;
};

__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& tm, int& tn) {
    const int per_group = p.group_m * p.tiles_n;
    const int g = tile / per_group;
    const int first_m = g * p.group_m;
    const int gsz = min(p.tiles_m - first_m, p.group_m);
    const int in = tile - g * per_group;
    tm = first_m + in % gsz;
    tn = in / gsz;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
    constexpr int kBStageBytes = BN * kBK * 2;
    constexpr int kStageBytes = kAStageBytes + kBStageBytes;
    constexpr uint32_t kTmemCols = 2 * BN;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * kAStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * kStageBytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* tmem_full = bars + 2 * STAGES;
    uint64_t* tmem_empty = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmem_full[a], 1);
            mbar_init(&tmem_empty[a], 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_tiles = p.tiles_m * p.tiles_n;
    const int num_kb = (p.K + kBK - 1) / kBK;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int tm, tn;
                tile_coords(p, tile, tm, tn);
                const int m0 = tm * kBM, n0 = tn * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_TMA_EMPTY)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[s], kStageBytes);
                    uint8_t* a_dst = sA + s * kAStageBytes;
                    uint8_t* b_dst = sB + s * kBStageBytes;
                    const int k0 = kb * kBK;
                    if (!p.a_mn) {
                        tma_load_2d(a_dst, &tmA, &full[s], k0, m0);
                    } else {
#pragma unroll
                        for (int c = 0; c < kBM / 64; ++c)
                            tma_load_2d(a_dst + c * (kBK * 128), &tmA, &full[s], m0 + c * 64, k0);
                    }
                    if (!p.b_mn) {
                        tma_load_2d(b_dst, &tmB, &full[s], k0, n0);
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c)
                            tma_load_2d(b_dst + c * (kBK * 128), &tmB, &full[s], n0 + c * 64, k0);
                    }
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
            if (!ok) {
                // Give copies still in flight time to land before the CTA's memory is released.
                for (int i = 0; i < 32; ++i) __nanosleep(50000);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer
            const uint32_t idesc = umma_idesc_bf16(kBM, BN, p.a_mn, p.b_mn);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int t = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
                const int acc = t & 1;
                const uint32_t acc_ph = (t >> 1) & 1;
                if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_TMEM_EMPTY)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&full[s], ph, abort_flag, p.status, CAI_DEV_TIMEOUT_TMA_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(sA + s * kAStageBytes);
                    const uint32_t b_base = smem_u32(sB + s * kBStageBytes);
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        const uint64_t adesc =
                            p.a_mn ? umma_smem_desc_sw128(a_base + k * (kUmmaK * 128), kBK * 128, 1024)
                                   : umma_smem_desc_sw128(a_base + k * (kUmmaK * 2), 0, 1024);
                        const uint64_t bdesc =
                            p.b_mn ? umma_smem_desc_sw128(b_base + k * (kUmmaK * 128), kBK * 128, 1024)
                                   : umma_smem_desc_sw128(b_base + k * (kUmmaK * 2), 0, 1024);
                        umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) umma_commit(&tmem_full[acc]);
            }
        }
    } else {
        // ---------------- epilogue warps: TMEM -> registers -> global
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        int t = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
            int tm, tn;
            tile_coords(p, tile, tm, tn);
            const int acc = t & 1;
            const uint32_t acc_ph = (t >> 1) & 1;
            if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag, p.status, CAI_DEV_TIMEOUT_TMEM_FULL)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const long long row = (long long)tm * kBM + q * 32 + lane;
            const bool row_ok = row < p.M;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32;
                tmem_ld_32x32(taddr, r);
                tmem_ld_wait();
                const int col0 = tn * BN + c * 32;
                if (!row_ok || col0 >= p.N) continue;
                const float alpha = p.alpha;
                if (p.epi == CAI_EPI_BF16 || p.epi == CAI_EPI_BF16_RESIDUAL) {
                    __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
                    const __nv_bfloat16* rrow =
                        p.epi == CAI_EPI_BF16_RESIDUAL
                            ? reinterpret_cast<const __nv_bfloat16*>(p.R) + row * p.ldr + col0
                            : nullptr;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (col0 + j * 8 >= p.N) break;
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j * 8 + e]) * alpha;
                        if (rrow) {
                            const uint4 rv = *reinterpret_cast<const uint4*>(rrow + j * 8);
                            v[0] += bf16_lo(rv.x); v[1] += bf16_hi(rv.x);
                            v[2] += bf16_lo(rv.y); v[3] += bf16_hi(rv.y);
                            v[4] += bf16_lo(rv.z); v[5] += bf16_hi(rv.z);
                            v[6] += bf16_lo(rv.w); v[7] += bf16_hi(rv.w);
                        }
                        uint4 o;
                        o.x = pack_bf16(v[0], v[1]);
                        o.y = pack_bf16(v[2], v[3]);
                        o.z = pack_bf16(v[4], v[5]);
                        o.w = pack_bf16(v[6], v[7]);
                        *reinterpret_cast<uint4*>(crow + j * 8) = o;
                    }
                } else {
                    float* crow = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
                    const bool accum = p.epi == CAI_EPI_F32_ACCUM;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (col0 + j * 4 >= p.N) break;
                        float4 o;
                        o.x = __uint_as_float(r[j * 4 + 0]) * alpha;
                        o.y = __uint_as_float(r[j * 4 + 1]) * alpha;
                        o.z = __uint_as_float(r[j * 4 + 2]) * alpha;
                        o.w = __uint_as_float(r[j * 4 + 3]) * alpha;
                        if (accum) {
                            const float4 old = *reinterpret_cast<const float4*>(crow + j * 4);
                            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                        }
                        *reinterpret_cast<float4*>(crow + j * 4) = o;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams& p, int sms,
                       cudaStream_t stream) {
    constexpr int smem_bytes = STAGES * (kAStageBytes + BN * kBK * 2) + 1024 + 256;
    static bool configured[64] = {};
    const int dev = current_device();
    if (!configured[dev & 63]) {
        if (cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem_bytes) != cudaSuccess) {
            set_last_error("cudaFuncSetAttribute(gemm) failed: %s", cudaGetErrorString(cudaGetLastError()));
            return CAI_K_CUDA;
        }
        configured[dev & 63] = true;
    }
    p.tiles_m = (p.M + kBM - 1) / kBM;
    p.tiles_n = (p.N + BN - 1) / BN;
    p.group_m = 8;
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sms ? tiles : sms;
    gemm_bf16_kernel<BN, STAGES><<<grid, kGemmThreads, smem_bytes, stream>>>(tmA, tmB, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_error("gemm launch failed: %s", cudaGetErrorString(e));
        return CAI_K_CUDA;
    }
    return CAI_K_OK;
}

}  // namespace cai

using namespace cai;

CAI_API int cai_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                          long long lda, long long ldb, long long ldc, long long ldr, int a_mn_major,
                          int b_mn_major, int epi, float alpha, int sm_limit, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return CAI_K_OK;
    if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 3) || epi < 0 || epi > CAI_EPI_BF16_RESIDUAL) {
        set_last_error("gemm: N, lda, ldb must be multiples of 8 (N=%d lda=%lld ldb=%lld ldc=%lld epi=%d)", N,
                       lda, ldb, ldc, epi);
        return CAI_K_BAD_ARG;
    }
    if ((epi == CAI_EPI_BF16 || epi == CAI_EPI_BF16_RESIDUAL) && (ldc & 7)) {
        set_last_error("gemm: bf16 output needs ldc %% 8 == 0");
        return CAI_K_BAD_ARG;
    }
    if (epi == CAI_EPI_BF16_RESIDUAL && (!R || (ldr & 7))) {
        set_last_error("gemm: residual epilogue needs R with ldr %% 8 == 0");
        return CAI_K_BAD_ARG;
    }
    const int dev = current_device();
    int sms = sm_count(dev);
    if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;

    // Tile width: fewer, wider tiles amortise the A operand better; narrower tiles quantise
    // into waves better when the output is small.
    auto cost = [&](int bn) {
        const long long tiles = (long long)((M + kBM - 1) / kBM) * ((N + bn - 1) / bn);
        const long long waves = (tiles + sms - 1) / sms;
        return (double)waves * bn * (bn == 128 ? 1.06 : 1.0);
    };
    const int BN = cost(256) <= cost(128) ? 256 : 128;

    CUtensorMap tmA, tmB;
    bool ok;
    if (!a_mn_major) ok = encode_tmap_2d(&tmA, A, M, K, lda, kBK, kBM, 2);
    else ok = encode_tmap_2d(&tmA, A, K, M, lda, 64, kBK, 2);
    if (!ok) return CAI_K_BAD_ARG;
    if (!b_mn_major) ok = encode_tmap_2d(&tmB, B, N, K, ldb, kBK, BN, 2);
    else ok = encode_tmap_2d(&tmB, B, K, N, ldb, 64, kBK, 2);
    if (!ok) return CAI_K_BAD_ARG;

    GemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.a_mn = a_mn_major ? 1 : 0;
    p.b_mn = b_mn_major ? 1 : 0;
    p.epi = epi;
    p.alpha = alpha;
    p.C = C; p.R = R;
    p.ldc = ldc; p.ldr = ldr;
    p.status = status_words(dev);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (BN == 256) return launch_gemm<256, 4>(tmA, tmB, p, sms, st);
    return launch_gemm<128, 6>(tmA, tmB, p, sms, st);
}
