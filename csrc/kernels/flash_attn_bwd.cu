// flash_attn_bwd.cu - causal grouped-query flash attention backward for sm_100a, head_dim 128.
//
// Three launches, all deterministic (no atomics):
//   1. attn_delta_kernel   delta[b,h,s] = sum_d dO * O                      (bandwidth bound)
//   2. attn_dkdv_kernel    one CTA per (kv tile, kv head, batch). It sweeps the query tiles at or
//                          below the diagonal of every query head of the group and accumulates
//                          dK and dV in tensor memory. Scores are computed transposed
//                          (S^T = K Q^T, dP^T = V dO^T) so that TMEM lanes are kv rows; the bf16
//                          P^T and dS^T are written back over S^T / dP^T and feed
//                          dV += P^T dO and dK += dS^T Q as A operands straight from TMEM.
//   3. attn_dq_kernel      one CTA per (q tile, head, batch): S = Q K^T, dP = dO V^T,
//                          dS -> TMEM, dQ += dS K.
// Q, K, V and dO tiles arrive by TMA from the packed activation; each shared-memory tile serves
// both as a K-major operand (for the score products) and as an MN-major operand (for the
// gradient products) through different UMMA descriptors, so nothing is transposed in memory.
//
// Replaces the reference's one-thread-per-query backward, which recomputes dp twice, scatters
// dK/dV with atomicAdd and never zeroes dq/dk/dv (src/cuda/cai_kernels.cu:110-143).
#include <math.h>

#include "attn_common.cuh"
#include "cai_kernels.h"
#include "host_common.h"
#include "sm100.cuh"

namespace cai {

constexpr int kAttnBwdThreads = 384;  // warp 0 TMA, warp 1 MMA, warps 4-11 compute (two groups split the columns)

struct AttnBwdParams {
    int B, S, nh, nkv;
    float scale, scale_log2;
    const float* lse;
    const float* delta;
    __nv_bfloat16* dqkv;
    int* status;
    // dK / dV with one CTA per QUERY head (small grids): the heads of a kv group take turns adding their
    // contribution to the group's dK / dV rows; chain[b][g][kv tile] counts the heads that are done.
    int split_heads;
    unsigned int* chain;
};

// chain counters of the head-split dK / dV kernel: one per (batch, kv group, kv tile).
// ONE array serves every call on a device: each call clears the slots it uses (stream-ordered memset) before
// its kernel, so two attention backwards that overlap on one GPU (different streams) would reset each other's
// counters. Calls that take the head-split path must therefore be ordered against each other; the executor
// issues them from one stream. A CTA of turn t waits (bounded) for the CTA of turn t - 1 of the same kv tile,
// which has a lower linear block id: with the grid no larger than the number of SMs every CTA is resident at
// once and the order of dispatch does not matter; the launcher only takes this path then.
constexpr size_t kAttnChainSlots = 65536;
__device__ unsigned int g_attn_chain[kAttnChainSlots];

__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int B, int S, int nh) {
    const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const long long total = static_cast<long long>(B) * S * nh;
    if (w >= total) return;
    const int h = w % nh;
    const long long row = w / nh;  // b*S + s
    const long long off = row * (static_cast<long long>(nh) * kAttnHD) + h * kAttnHD + lane * 4;
    const uint2 a = *reinterpret_cast<const uint2*>(out + off);
    const uint2 d = *reinterpret_cast<const uint2*>(dout + off);
    float s = bf16_lo(a.x) * bf16_lo(d.x) + bf16_hi(a.x) * bf16_hi(d.x) + bf16_lo(a.y) * bf16_lo(d.y) +
              bf16_hi(a.y) * bf16_hi(d.y);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
        const int b = row / S, sidx = row % S;
        delta[(static_cast<long long>(b) * nh + h) * S + sidx] = s;
    }
}

__device__ __forceinline__ void bar_sync_compute() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Store one finished 128x128 fp32 accumulator (TMEM) as bf16 rows of the packed gradient buffer.
__device__ __forceinline__ void store_acc_bf16(uint32_t tacc, __nv_bfloat16* dst_row, int c_lo = 0, int c_hi = 4) {
#pragma unroll 1
    for (int c = c_lo; c < c_hi; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tacc + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(v[j4 * 8 + 0]), __uint_as_float(v[j4 * 8 + 1]));
            o.y = pack_bf16(__uint_as_float(v[j4 * 8 + 2]), __uint_as_float(v[j4 * 8 + 3]));
            o.z = pack_bf16(__uint_as_float(v[j4 * 8 + 4]), __uint_as_float(v[j4 * 8 + 5]));
            o.w = pack_bf16(__uint_as_float(v[j4 * 8 + 6]), __uint_as_float(v[j4 * 8 + 7]));
            *reinterpret_cast<uint4*>(dst_row + c * 32 + j4 * 8) = o;
        }
    }
}

// The same, added to what the rows already hold (bf16 read-modify-write).
__device__ __forceinline__ void add_acc_bf16(uint32_t tacc, __nv_bfloat16* dst_row) {
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tacc + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
            const uint4 old = *reinterpret_cast<const uint4*>(dst_row + c * 32 + j4 * 8);
            uint4 o;
            o.x = pack_bf16(__uint_as_float(v[j4 * 8 + 0]) + bf16_lo(old.x), __uint_as_float(v[j4 * 8 + 1]) + bf16_hi(old.x));
            o.y = pack_bf16(__uint_as_float(v[j4 * 8 + 2]) + bf16_lo(old.y), __uint_as_float(v[j4 * 8 + 3]) + bf16_hi(old.y));
            o.z = pack_bf16(__uint_as_float(v[j4 * 8 + 4]) + bf16_lo(old.z), __uint_as_float(v[j4 * 8 + 5]) + bf16_hi(old.z));
            o.w = pack_bf16(__uint_as_float(v[j4 * 8 + 6]) + bf16_lo(old.w), __uint_as_float(v[j4 * 8 + 7]) + bf16_hi(old.w));
            *reinterpret_cast<uint4*>(dst_row + c * 32 + j4 * 8) = o;
        }
    }
}

// ---------------------------------------------------------------------------- dK / dV
__global__ void __launch_bounds__(kAttnBwdThreads, 1)
attn_dkdv_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                 const AttnBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;
    uint8_t* sV = smem + kAttnTileBytes;
    uint8_t* sQ = smem + 2 * kAttnTileBytes;   // 2 stages
    uint8_t* sdO = smem + 4 * kAttnTileBytes;  // 2 stages
    float* sL = reinterpret_cast<float*>(smem + 6 * kAttnTileBytes);  // [2][128] lse * log2e
    float* sD = sL + 256;                                              // [2][128] delta
    uint64_t* bars = reinterpret_cast<uint64_t*>(sD + 256);
    uint64_t* kv_full = bars;
    uint64_t* qdo_full = bars + 1;
    uint64_t* qdo_empty = bars + 3;
    uint64_t* sdp_full = bars + 5;
    uint64_t* pds_ready = bars + 6;
    uint64_t* final_bar = bars + 7;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // linear dispatch order -> (kv tile slowest, heaviest first; heads and batch fastest)
    const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    const int heads_all = gridDim.y * gridDim.z;
    const int j = lin / heads_all;  // kv tile
    const int ysel = (lin % heads_all) % gridDim.y, b = (lin % heads_all) / gridDim.y;
    const int rep = p.nh / p.nkv;
    // grid.y is kv groups (a CTA sweeps the group's query heads) or, with split_heads, query heads
    const int g = p.split_heads ? ysel / rep : ysel;
    const int h_first = p.split_heads ? ysel : g * rep;
    const int turn = p.split_heads ? ysel - g * rep : 0;   // my place in the group's accumulation chain
    const int nq = p.S / kAttnTile;
    const int per_head = nq - j;          // query tiles at or below the diagonal
    const int iters = (p.split_heads ? 1 : rep) * per_head;
    const int row_base = b * p.S;
    const int col_k = (p.nh + g) * kAttnHD, col_v = (p.nh + p.nkv + g) * kAttnHD;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_qkv);
        tma_prefetch_desc(&tm_do);
        mbar_init(kv_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&qdo_full[i], 1);
            mbar_init(&qdo_empty[i], 1);
        }
        mbar_init(sdp_full, 1);
        mbar_init(pds_ready, 256);
        mbar_init(final_bar, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 384;

    if (warp == 0) {
        if (lane == 0) {
            const int kv_row = row_base + j * kAttnTile;
            mbar_expect_tx(kv_full, 2 * kAttnTileBytes);
            tma_load_2d(sK, &tm_qkv, kv_full, col_k, kv_row);
            tma_load_2d(sK + kAttnSub, &tm_qkv, kv_full, col_k + 64, kv_row);
            tma_load_2d(sV, &tm_qkv, kv_full, col_v, kv_row);
            tma_load_2d(sV + kAttnSub, &tm_qkv, kv_full, col_v + 64, kv_row);
            bool ok = true;
            for (int it = 0; it < iters && ok; ++it) {
                const int slot = it & 1;
                const uint32_t ph = (it >> 1) & 1;
                const int h = h_first + it / per_head;
                const int q_row = row_base + (j + it % per_head) * kAttnTile;
                if (!mbar_wait(&qdo_empty[slot], ph ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                mbar_expect_tx(&qdo_full[slot], 2 * kAttnTileBytes);
                uint8_t* q = sQ + slot * kAttnTileBytes;
                uint8_t* d = sdO + slot * kAttnTileBytes;
                tma_load_2d(q, &tm_qkv, &qdo_full[slot], h * kAttnHD, q_row);
                tma_load_2d(q + kAttnSub, &tm_qkv, &qdo_full[slot], h * kAttnHD + 64, q_row);
                tma_load_2d(d, &tm_do, &qdo_full[slot], h * kAttnHD, q_row);
                tma_load_2d(d + kAttnSub, &tm_do, &qdo_full[slot], h * kAttnHD + 64, q_row);
            }
            if (!ok)
                for (int i = 0; i < 32; ++i) __nanosleep(50000);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_kk = umma_idesc_bf16(128, 128, 0, 0);
            const uint32_t idesc_mn = umma_idesc_bf16(128, 128, 0, 1);
            const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aD = smem_u32(sdO);
            bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN);
            for (int it = 0; it < iters && ok; ++it) {
                const int slot = it & 1;
                const uint32_t ph = (it >> 1) & 1;
                if (!mbar_wait(&qdo_full[slot], ph, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                tc_fence_after();
                issue_qk(tS, aK, aQ + slot * kAttnTileBytes, idesc_kk);    // S^T  = K Q^T
                issue_qk(tdP, aV, aD + slot * kAttnTileBytes, idesc_kk);   // dP^T = V dO^T
                umma_commit(sdp_full);
                if (!mbar_wait(pds_ready, it & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                tc_fence_after();
                issue_pv(tdV, tS, aD + slot * kAttnTileBytes, idesc_mn, it > 0);   // dV += P^T dO
                issue_pv(tdK, tdP, aQ + slot * kAttnTileBytes, idesc_mn, it > 0);  // dK += dS^T Q
                umma_commit(&qdo_empty[slot]);
            }
            if (ok) umma_commit(final_bar);
        }
    } else if (warp >= 4) {
        const int r = (warp & 3) * 32 + lane;  // kv row inside the tile == TMEM lane
        const int half = warp >= 8 ? 1 : 0;    // which 64 query columns this warp group handles
        const uint32_t lane_bits = static_cast<uint32_t>((warp & 3) * 32) << 16;
        bool ok = true;
        for (int it = 0; it < iters; ++it) {
            const int h = h_first + it / per_head;
            const int i = j + it % per_head;
            const int buf = it & 1;
            const long long vec = (static_cast<long long>(b) * p.nh + h) * p.S + i * kAttnTile + r;
            if (half == 0) sL[buf * 128 + r] = p.lse[vec] * 1.4426950408889634f;
            else sD[buf * 128 + r] = p.delta[vec];
            bar_sync_compute();
            if (!mbar_wait(sdp_full, it & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
            tc_fence_after();
            const bool diag = (i == j);
            const float* L = sL + buf * 128;
            const float* D = sD + buf * 128;
            // Both warp groups read their score columns first and keep the bf16 results in registers;
            // only after every thread has finished reading are P^T / dS^T written back over S^T / dP^T
            // (the packed output of the upper columns lands where the lower columns were read from).
            uint32_t pk[2][16], dk[2][16];
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int c = half * 2 + cc;
                uint32_t s[32], dp[32];
                tmem_ld_32x32(tS + lane_bits + c * 32, s);
                tmem_ld_32x32(tdP + lane_bits + c * 32, dp);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const int q0 = c * 32 + e;
                    float p0 = fast_exp2(__uint_as_float(s[e]) * p.scale_log2 - L[q0]);
                    float p1 = fast_exp2(__uint_as_float(s[e + 1]) * p.scale_log2 - L[q0 + 1]);
                    if (diag) {  // key (row r) may not lie after the query (column)
                        if (r > q0) p0 = 0.f;
                        if (r > q0 + 1) p1 = 0.f;
                    }
                    const float d0 = p0 * (__uint_as_float(dp[e]) - D[q0]) * p.scale;
                    const float d1 = p1 * (__uint_as_float(dp[e + 1]) - D[q0 + 1]) * p.scale;
                    pk[cc][e >> 1] = pack_bf16(p0, p1);
                    dk[cc][e >> 1] = pack_bf16(d0, d1);
                }
            }
            tc_fence_before();
            bar_sync_compute();
            tc_fence_after();
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int c = half * 2 + cc;
                tmem_st_32x16(tS + lane_bits + c * 16, pk[cc]);
                tmem_st_32x16(tdP + lane_bits + c * 16, dk[cc]);
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(pds_ready);
        }
        if (ok && mbar_wait(final_bar, 0, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) {
            tc_fence_after();
            const long long grow = static_cast<long long>(row_base) + j * kAttnTile + r;
            const long long ld = static_cast<long long>(p.nh + 2 * p.nkv) * kAttnHD;
            __nv_bfloat16* dst = p.dqkv + grow * ld + (half == 0 ? col_k : col_v);
            const uint32_t tacc = (half == 0 ? tdK : tdV) + lane_bits;
            if (!p.split_heads) {
                store_acc_bf16(tacc, dst);
            } else {
                // heads of the group add in turn: wait (bounded) until the heads before me are done
                unsigned int* cnt = p.chain + (static_cast<long long>(b) * p.nkv + g) * nq + j;
                bool go = true;
                if (turn > 0) {
                    go = false;
                    for (uint32_t spin = 0; spin < kSpinLimit && !go; ++spin) {
                        unsigned int v;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
                        go = v >= static_cast<unsigned int>(turn);
                        if (!go && spin > 16) __nanosleep(200);
                    }
                    if (!go) atomicCAS(p.status, 0, CAI_DEV_TIMEOUT_ATTN);
                }
                if (go) {
                    if (turn == 0) store_acc_bf16(tacc, dst);
                    else add_acc_bf16(tacc, dst);
                }
                __threadfence();
                bar_sync_compute();
                if (threadIdx.x == 128) {   // first compute thread: everyone's rows are written and fenced
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(cnt), "r"(static_cast<unsigned int>(turn + 1)) : "memory");
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---------------------------------------------------------------------------- dQ
__global__ void __launch_bounds__(kAttnBwdThreads, 1)
attn_dq_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
               const AttnBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sdO = smem + kAttnTileBytes;
    uint8_t* sK = smem + 2 * kAttnTileBytes;  // 2 stages
    uint8_t* sV = smem + 4 * kAttnTileBytes;  // 2 stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kAttnTileBytes);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;
    uint64_t* kv_empty = bars + 3;
    uint64_t* sdp_full = bars + 5;
    uint64_t* ds_ready = bars + 6;
    uint64_t* final_bar = bars + 7;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    const int heads_all = gridDim.y * gridDim.z;
    const int i = gridDim.x - 1 - lin / heads_all;  // q tile, heaviest first across all heads
    const int h = (lin % heads_all) % gridDim.y, b = (lin % heads_all) / gridDim.y;
    const int g = h / (p.nh / p.nkv);
    const int n = i + 1;
    const int row_base = b * p.S;
    const int col_q = h * kAttnHD, col_k = (p.nh + g) * kAttnHD, col_v = (p.nh + p.nkv + g) * kAttnHD;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_qkv);
        tma_prefetch_desc(&tm_do);
        mbar_init(q_full, 1);
        for (int k = 0; k < 2; ++k) {
            mbar_init(&kv_full[k], 1);
            mbar_init(&kv_empty[k], 1);
        }
        mbar_init(sdp_full, 1);
        mbar_init(ds_ready, 256);
        mbar_init(final_bar, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdQ = tmem_base + 256;

    if (warp == 0) {
        if (lane == 0) {
            const int q_row = row_base + i * kAttnTile;
            mbar_expect_tx(q_full, 2 * kAttnTileBytes);
            tma_load_2d(sQ, &tm_qkv, q_full, col_q, q_row);
            tma_load_2d(sQ + kAttnSub, &tm_qkv, q_full, col_q + 64, q_row);
            tma_load_2d(sdO, &tm_do, q_full, col_q, q_row);
            tma_load_2d(sdO + kAttnSub, &tm_do, q_full, col_q + 64, q_row);
            bool ok = true;
            for (int j = 0; j < n && ok; ++j) {
                const int slot = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                const int kv_row = row_base + j * kAttnTile;
                if (!mbar_wait(&kv_empty[slot], ph ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                mbar_expect_tx(&kv_full[slot], 2 * kAttnTileBytes);
                uint8_t* k = sK + slot * kAttnTileBytes;
                uint8_t* v = sV + slot * kAttnTileBytes;
                tma_load_2d(k, &tm_qkv, &kv_full[slot], col_k, kv_row);
                tma_load_2d(k + kAttnSub, &tm_qkv, &kv_full[slot], col_k + 64, kv_row);
                tma_load_2d(v, &tm_qkv, &kv_full[slot], col_v, kv_row);
                tma_load_2d(v + kAttnSub, &tm_qkv, &kv_full[slot], col_v + 64, kv_row);
            }
            if (!ok)
                for (int k = 0; k < 32; ++k) __nanosleep(50000);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_kk = umma_idesc_bf16(128, 128, 0, 0);
            const uint32_t idesc_mn = umma_idesc_bf16(128, 128, 0, 1);
            const uint32_t aQ = smem_u32(sQ), aD = smem_u32(sdO), aK = smem_u32(sK), aV = smem_u32(sV);
            bool ok = mbar_wait(q_full, 0, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN);
            for (int j = 0; j < n && ok; ++j) {
                const int slot = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                if (!mbar_wait(&kv_full[slot], ph, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                tc_fence_after();
                issue_qk(tS, aQ, aK + slot * kAttnTileBytes, idesc_kk);    // S  = Q K^T
                issue_qk(tdP, aD, aV + slot * kAttnTileBytes, idesc_kk);   // dP = dO V^T
                umma_commit(sdp_full);
                if (!mbar_wait(ds_ready, j & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                tc_fence_after();
                issue_pv(tdQ, tdP, aK + slot * kAttnTileBytes, idesc_mn, j > 0);  // dQ += dS K
                umma_commit(&kv_empty[slot]);
            }
            if (ok) umma_commit(final_bar);
        }
    } else if (warp >= 4) {
        const int r = (warp & 3) * 32 + lane;  // q row inside the tile
        const int half = warp >= 8 ? 1 : 0;    // which 64 key columns this warp group handles
        const uint32_t lane_bits = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const long long vec = (static_cast<long long>(b) * p.nh + h) * p.S + i * kAttnTile + r;
        const float lse2 = p.lse[vec] * 1.4426950408889634f;
        const float dl = p.delta[vec];
        bool ok = true;
        for (int j = 0; j < n; ++j) {
            if (!mbar_wait(sdp_full, j & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
            tc_fence_after();
            const bool diag = (j == i);
            uint32_t dk[2][16];
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int c = half * 2 + cc;
                uint32_t s[32], dp[32];
                tmem_ld_32x32(tS + lane_bits + c * 32, s);
                tmem_ld_32x32(tdP + lane_bits + c * 32, dp);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const int k0 = c * 32 + e;
                    float p0 = fast_exp2(__uint_as_float(s[e]) * p.scale_log2 - lse2);
                    float p1 = fast_exp2(__uint_as_float(s[e + 1]) * p.scale_log2 - lse2);
                    if (diag) {
                        if (k0 > r) p0 = 0.f;
                        if (k0 + 1 > r) p1 = 0.f;
                    }
                    dk[cc][e >> 1] = pack_bf16(p0 * (__uint_as_float(dp[e]) - dl) * p.scale,
                                               p1 * (__uint_as_float(dp[e + 1]) - dl) * p.scale);
                }
            }
            // dS is written back over dP only after both warp groups have read their dP columns
            tc_fence_before();
            bar_sync_compute();
            tc_fence_after();
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) tmem_st_32x16(tdP + lane_bits + (half * 2 + cc) * 16, dk[cc]);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(ds_ready);
        }
        if (ok && mbar_wait(final_bar, 0, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) {
            tc_fence_after();
            const long long grow = static_cast<long long>(row_base) + i * kAttnTile + r;
            const long long ld = static_cast<long long>(p.nh + 2 * p.nkv) * kAttnHD;
            store_acc_bf16(tdQ + lane_bits, p.dqkv + grow * ld + col_q, half * 2, half * 2 + 2);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}


// ---------------------------------------------------------------------------- pipelined forms
// The kernels above keep one 128 x 128 score tile in flight: the MMAs of a step wait for the exponentials of the
// same step and the tensor pipe idles two thirds of the time. The forms below split every step into two 64-column
// half steps with their own S / dP accumulators (64 TMEM columns each, the same 512 columns in total) and stream
// the swept operand in 64-row half tiles through four shared-memory stages. The MMA thread runs the score products
// of half step u + 2 right behind the gradient products of half step u, so the tensor pipe works on one half while
// the compute warps work on the other. A warp group writes its bf16 results over the first half of the 32 fp32
// columns it has just read (no other warp reads those), so a half step needs no barrier between the groups; the
// A operand of the gradient products is addressed in two 16-column pieces.
constexpr int kAttnPipeStages = 4;
constexpr int kAttnPipeStageBytes = 2 * kAttnHalfBytes;  // two 64-row operands per stage (Q + dO, or K + V)

struct AttnPipeSmem {
    uint8_t* fixed0;   // dK/dV: K     dQ: Q
    uint8_t* fixed1;   // dK/dV: V     dQ: dO
    uint8_t* stages;   // 4 x (64-row operand pair)
    float* sL;
    float* sD;
    uint64_t* fixed_full;
    uint64_t* st_full;
    uint64_t* st_empty;
    uint64_t* sdp_full;
    uint64_t* out_ready;
    uint64_t* final_bar;
    uint32_t* tmem_slot;
    volatile int* abort_flag;
};

__device__ __forceinline__ AttnPipeSmem attn_pipe_carve(uint8_t* smem_raw) {
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    AttnPipeSmem m;
    m.fixed0 = smem;
    m.fixed1 = smem + kAttnTileBytes;
    m.stages = smem + 2 * kAttnTileBytes;
    m.sL = reinterpret_cast<float*>(smem + 2 * kAttnTileBytes + kAttnPipeStages * kAttnPipeStageBytes);
    m.sD = m.sL + 256;
    uint64_t* bars = reinterpret_cast<uint64_t*>(m.sD + 256);
    m.fixed_full = bars;
    m.st_full = bars + 1;
    m.st_empty = bars + 5;
    m.sdp_full = bars + 9;
    m.out_ready = bars + 11;
    m.final_bar = bars + 13;
    m.tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
    m.abort_flag = reinterpret_cast<volatile int*>(m.tmem_slot + 1);
    return m;
}

__device__ __forceinline__ void attn_pipe_init(const AttnPipeSmem& m) {
    mbar_init(m.fixed_full, 1);
    for (int i = 0; i < kAttnPipeStages; ++i) {
        mbar_init(&m.st_full[i], 1);
        mbar_init(&m.st_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
        mbar_init(&m.sdp_full[i], 1);
        mbar_init(&m.out_ready[i], 256);
    }
    mbar_init(m.final_bar, 1);
    *m.abort_flag = 0;
    mbar_fence_init();
}

__global__ void __launch_bounds__(kAttnBwdThreads, 1)
attn_dkdv_pipe_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_qkv64,
                      const __grid_constant__ CUtensorMap tm_do64, const AttnBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    const AttnPipeSmem m = attn_pipe_carve(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    const int heads_all = gridDim.y * gridDim.z;
    const int j = lin / heads_all;  // kv tile, heaviest first
    const int ysel = (lin % heads_all) % gridDim.y, b = (lin % heads_all) / gridDim.y;
    const int rep = p.nh / p.nkv;
    const int g = p.split_heads ? ysel / rep : ysel;
    const int h_first = p.split_heads ? ysel : g * rep;
    const int turn = p.split_heads ? ysel - g * rep : 0;
    const int nq = p.S / kAttnTile;
    const int per_head = nq - j;
    const int iters = (p.split_heads ? 1 : rep) * per_head;
    const int total = 2 * iters;  // half steps
    const int row_base = b * p.S;
    const int col_k = (p.nh + g) * kAttnHD, col_v = (p.nh + p.nkv + g) * kAttnHD;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_qkv);
        tma_prefetch_desc(&tm_qkv64);
        tma_prefetch_desc(&tm_do64);
        attn_pipe_init(m);
    }
    if (warp == 1) {
        tmem_alloc(m.tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *m.tmem_slot;
    // half step s: S^T at tmem_base + s * 128, dP^T 64 columns behind it
    const uint32_t tdV = tmem_base + 256, tdK = tmem_base + 384;

    if (warp == 0) {
        if (lane == 0) {
            const int kv_row = row_base + j * kAttnTile;
            mbar_expect_tx(m.fixed_full, 2 * kAttnTileBytes);
            tma_load_2d(m.fixed0, &tm_qkv, m.fixed_full, col_k, kv_row);
            tma_load_2d(m.fixed0 + kAttnSub, &tm_qkv, m.fixed_full, col_k + 64, kv_row);
            tma_load_2d(m.fixed1, &tm_qkv, m.fixed_full, col_v, kv_row);
            tma_load_2d(m.fixed1 + kAttnSub, &tm_qkv, m.fixed_full, col_v + 64, kv_row);
            bool ok = true;
            for (int u = 0; u < total && ok; ++u) {
                const int st = u & 3, it = u >> 1;
                const uint32_t ph = (u >> 2) & 1;
                const int h = h_first + it / per_head;
                const int q_row = row_base + (j + it % per_head) * kAttnTile + (u & 1) * 64;
                if (!mbar_wait(&m.st_empty[st], ph ^ 1, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                mbar_expect_tx(&m.st_full[st], kAttnPipeStageBytes);
                uint8_t* q = m.stages + st * kAttnPipeStageBytes;
                uint8_t* d = q + kAttnHalfBytes;
                tma_load_2d(q, &tm_qkv64, &m.st_full[st], h * kAttnHD, q_row);
                tma_load_2d(q + kAttnHalfSub, &tm_qkv64, &m.st_full[st], h * kAttnHD + 64, q_row);
                tma_load_2d(d, &tm_do64, &m.st_full[st], h * kAttnHD, q_row);
                tma_load_2d(d + kAttnHalfSub, &tm_do64, &m.st_full[st], h * kAttnHD + 64, q_row);
            }
            if (!ok)
                for (int i = 0; i < 32; ++i) __nanosleep(50000);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_n64 = umma_idesc_bf16(128, 64, 0, 0);
            const uint32_t idesc_mn = umma_idesc_bf16(128, 128, 0, 1);
            const uint32_t aK = smem_u32(m.fixed0), aV = smem_u32(m.fixed1), aSt = smem_u32(m.stages);
            bool ok = mbar_wait(m.fixed_full, 0, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN);
            // score products of half step u: S^T = K Q_u^T, dP^T = V dO_u^T
            auto scores = [&](int u) -> bool {
                const int st = u & 3, s = u & 1;
                if (!mbar_wait(&m.st_full[st], (u >> 2) & 1, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) return false;
                tc_fence_after();
                const uint32_t q = aSt + st * kAttnPipeStageBytes, d = q + kAttnHalfBytes;
                issue_qk_n64(tmem_base + s * 128, aK, q, idesc_n64);
                issue_qk_n64(tmem_base + s * 128 + 64, aV, d, idesc_n64);
                umma_commit(&m.sdp_full[s]);
                return true;
            };
            if (ok) ok = scores(0);
            if (ok) ok = scores(1);
            for (int u = 0; u < total && ok; ++u) {
                const int st = u & 3, s = u & 1;
                if (!mbar_wait(&m.out_ready[s], (u >> 1) & 1, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                tc_fence_after();
                const uint32_t q = aSt + st * kAttnPipeStageBytes, d = q + kAttnHalfBytes;
                issue_pv_k64(tdV, tmem_base + s * 128, d, idesc_mn, u > 0);       // dV += P^T dO
                issue_pv_k64(tdK, tmem_base + s * 128 + 64, q, idesc_mn, u > 0);  // dK += dS^T Q
                umma_commit(&m.st_empty[st]);
                if (u + 2 < total) ok = scores(u + 2);
            }
            if (ok) umma_commit(m.final_bar);
        }
    } else if (warp >= 4) {
        const int r = (warp & 3) * 32 + lane;  // kv row inside the tile == TMEM lane
        const int half = warp >= 8 ? 1 : 0;    // which 32 of a half step's 64 query columns
        const uint32_t lane_bits = static_cast<uint32_t>((warp & 3) * 32) << 16;
        bool ok = true;
        for (int it = 0; it < iters && ok; ++it) {
            const int h = h_first + it / per_head;
            const int i = j + it % per_head;
            const int buf = it & 1;
            const long long vec = (static_cast<long long>(b) * p.nh + h) * p.S + i * kAttnTile + r;
            if (half == 0) m.sL[buf * 128 + r] = p.lse[vec] * 1.4426950408889634f;
            else m.sD[buf * 128 + r] = p.delta[vec];
            bar_sync_compute();
            const bool diag = (i == j);
#pragma unroll 1
            for (int s = 0; s < 2; ++s) {
                if (!mbar_wait(&m.sdp_full[s], it & 1, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                tc_fence_after();
                const int qb = s * 64 + half * 32;  // first query column of this thread's chunk
                const uint32_t tS = tmem_base + lane_bits + s * 128 + half * 32;
                const uint32_t tdP = tS + 64;
                const float4* L4 = reinterpret_cast<const float4*>(m.sL + buf * 128 + qb);
                const float4* D4 = reinterpret_cast<const float4*>(m.sD + buf * 128 + qb);
                uint32_t sv[32], dp[32], pk[16], dk[16];
                tmem_ld_32x32(tS, sv);
                tmem_ld_32x32(tdP, dp);
                tmem_ld_wait();
#pragma unroll
                for (int e4 = 0; e4 < 8; ++e4) {
                    const float4 l = L4[e4], dl = D4[e4];
                    const float ls[4] = {l.x, l.y, l.z, l.w}, ds[4] = {dl.x, dl.y, dl.z, dl.w};
                    float pr[4], dsv[4];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const int e = e4 * 4 + t;
                        float pv = fast_exp2(__uint_as_float(sv[e]) * p.scale_log2 - ls[t]);
                        if (diag && r > qb + e) pv = 0.f;  // key (row r) may not lie after the query (column)
                        pr[t] = pv;
                        dsv[t] = pv * (__uint_as_float(dp[e]) - ds[t]) * p.scale;
                    }
                    pk[e4 * 2] = pack_bf16(pr[0], pr[1]);
                    pk[e4 * 2 + 1] = pack_bf16(pr[2], pr[3]);
                    dk[e4 * 2] = pack_bf16(dsv[0], dsv[1]);
                    dk[e4 * 2 + 1] = pack_bf16(dsv[2], dsv[3]);
                }
                tmem_st_32x16(tS, pk);
                tmem_st_32x16(tdP, dk);
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(&m.out_ready[s]);
            }
        }
        if (ok && mbar_wait(m.final_bar, 0, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) {
            tc_fence_after();
            const long long grow = static_cast<long long>(row_base) + j * kAttnTile + r;
            const long long ld = static_cast<long long>(p.nh + 2 * p.nkv) * kAttnHD;
            __nv_bfloat16* dst = p.dqkv + grow * ld + (half == 0 ? col_k : col_v);
            const uint32_t tacc = (half == 0 ? tdK : tdV) + lane_bits;
            if (!p.split_heads) {
                store_acc_bf16(tacc, dst);
            } else {
                unsigned int* cnt = p.chain + (static_cast<long long>(b) * p.nkv + g) * nq + j;
                bool go = true;
                if (turn > 0) {
                    go = false;
                    for (uint32_t spin = 0; spin < kSpinLimit && !go; ++spin) {
                        unsigned int v;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
                        go = v >= static_cast<unsigned int>(turn);
                        if (!go && spin > 16) __nanosleep(200);
                    }
                    if (!go) atomicCAS(p.status, 0, CAI_DEV_TIMEOUT_ATTN);
                }
                if (go) {
                    if (turn == 0) store_acc_bf16(tacc, dst);
                    else add_acc_bf16(tacc, dst);
                }
                __threadfence();
                bar_sync_compute();
                if (threadIdx.x == 128) {
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(cnt), "r"(static_cast<unsigned int>(turn + 1)) : "memory");
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

__global__ void __launch_bounds__(kAttnBwdThreads, 1)
attn_dq_pipe_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_qkv64, const AttnBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    const AttnPipeSmem m = attn_pipe_carve(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    const int heads_all = gridDim.y * gridDim.z;
    const int i = gridDim.x - 1 - lin / heads_all;  // q tile, heaviest first across all heads
    const int h = (lin % heads_all) % gridDim.y, b = (lin % heads_all) / gridDim.y;
    const int g = h / (p.nh / p.nkv);
    const int total = 2 * (i + 1);  // half steps: 64 keys each
    const int row_base = b * p.S;
    const int col_q = h * kAttnHD, col_k = (p.nh + g) * kAttnHD, col_v = (p.nh + p.nkv + g) * kAttnHD;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_qkv);
        tma_prefetch_desc(&tm_do);
        tma_prefetch_desc(&tm_qkv64);
        attn_pipe_init(m);
    }
    if (warp == 1) {
        tmem_alloc(m.tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *m.tmem_slot;
    const uint32_t tdQ = tmem_base + 256;

    if (warp == 0) {
        if (lane == 0) {
            const int q_row = row_base + i * kAttnTile;
            mbar_expect_tx(m.fixed_full, 2 * kAttnTileBytes);
            tma_load_2d(m.fixed0, &tm_qkv, m.fixed_full, col_q, q_row);
            tma_load_2d(m.fixed0 + kAttnSub, &tm_qkv, m.fixed_full, col_q + 64, q_row);
            tma_load_2d(m.fixed1, &tm_do, m.fixed_full, col_q, q_row);
            tma_load_2d(m.fixed1 + kAttnSub, &tm_do, m.fixed_full, col_q + 64, q_row);
            bool ok = true;
            for (int u = 0; u < total && ok; ++u) {
                const int st = u & 3;
                const uint32_t ph = (u >> 2) & 1;
                const int kv_row = row_base + u * 64;
                if (!mbar_wait(&m.st_empty[st], ph ^ 1, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                mbar_expect_tx(&m.st_full[st], kAttnPipeStageBytes);
                uint8_t* k = m.stages + st * kAttnPipeStageBytes;
                uint8_t* v = k + kAttnHalfBytes;
                tma_load_2d(k, &tm_qkv64, &m.st_full[st], col_k, kv_row);
                tma_load_2d(k + kAttnHalfSub, &tm_qkv64, &m.st_full[st], col_k + 64, kv_row);
                tma_load_2d(v, &tm_qkv64, &m.st_full[st], col_v, kv_row);
                tma_load_2d(v + kAttnHalfSub, &tm_qkv64, &m.st_full[st], col_v + 64, kv_row);
            }
            if (!ok)
                for (int k = 0; k < 32; ++k) __nanosleep(50000);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_n64 = umma_idesc_bf16(128, 64, 0, 0);
            const uint32_t idesc_mn = umma_idesc_bf16(128, 128, 0, 1);
            const uint32_t aQ = smem_u32(m.fixed0), aD = smem_u32(m.fixed1), aSt = smem_u32(m.stages);
            bool ok = mbar_wait(m.fixed_full, 0, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN);
            auto scores = [&](int u) -> bool {   // S = Q K_u^T, dP = dO V_u^T
                const int st = u & 3, s = u & 1;
                if (!mbar_wait(&m.st_full[st], (u >> 2) & 1, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) return false;
                tc_fence_after();
                const uint32_t k = aSt + st * kAttnPipeStageBytes, v = k + kAttnHalfBytes;
                issue_qk_n64(tmem_base + s * 128, aQ, k, idesc_n64);
                issue_qk_n64(tmem_base + s * 128 + 64, aD, v, idesc_n64);
                umma_commit(&m.sdp_full[s]);
                return true;
            };
            if (ok) ok = scores(0);
            if (ok) ok = scores(1);
            for (int u = 0; u < total && ok; ++u) {
                const int st = u & 3, s = u & 1;
                if (!mbar_wait(&m.out_ready[s], (u >> 1) & 1, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                tc_fence_after();
                issue_pv_k64(tdQ, tmem_base + s * 128 + 64, aSt + st * kAttnPipeStageBytes, idesc_mn, u > 0);  // dQ += dS K
                umma_commit(&m.st_empty[st]);
                if (u + 2 < total) ok = scores(u + 2);
            }
            if (ok) umma_commit(m.final_bar);
        }
    } else if (warp >= 4) {
        const int r = (warp & 3) * 32 + lane;  // q row inside the tile
        const int half = warp >= 8 ? 1 : 0;    // which 32 of a half step's 64 key columns
        const uint32_t lane_bits = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const long long vec = (static_cast<long long>(b) * p.nh + h) * p.S + i * kAttnTile + r;
        const float lse2 = p.lse[vec] * 1.4426950408889634f;
        const float dl = p.delta[vec];
        bool ok = true;
#pragma unroll 1
        for (int u = 0; u < total; ++u) {
            const int s = u & 1;
            if (!mbar_wait(&m.sdp_full[s], (u >> 1) & 1, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
            tc_fence_after();
            const bool diag = (u >> 1) == i;
            const int kb = s * 64 + half * 32;  // first key column (inside the 128-key tile) of this thread's chunk
            const uint32_t tS = tmem_base + lane_bits + s * 128 + half * 32;
            const uint32_t tdP = tS + 64;
            uint32_t sv[32], dp[32], dk[16];
            tmem_ld_32x32(tS, sv);
            tmem_ld_32x32(tdP, dp);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                float p0 = fast_exp2(__uint_as_float(sv[e]) * p.scale_log2 - lse2);
                float p1 = fast_exp2(__uint_as_float(sv[e + 1]) * p.scale_log2 - lse2);
                if (diag) {
                    if (kb + e > r) p0 = 0.f;
                    if (kb + e + 1 > r) p1 = 0.f;
                }
                dk[e >> 1] = pack_bf16(p0 * (__uint_as_float(dp[e]) - dl) * p.scale,
                                       p1 * (__uint_as_float(dp[e + 1]) - dl) * p.scale);
            }
            tmem_st_32x16(tdP, dk);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&m.out_ready[s]);
        }
        if (ok && mbar_wait(m.final_bar, 0, m.abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) {
            tc_fence_after();
            const long long grow = static_cast<long long>(row_base) + i * kAttnTile + r;
            const long long ld = static_cast<long long>(p.nh + 2 * p.nkv) * kAttnHD;
            store_acc_bf16(tdQ + lane_bits, p.dqkv + grow * ld + col_q, half * 2, half * 2 + 2);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace cai

using namespace cai;

CAI_API int cai_flash_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                               void* dqkv, int B, int S, int nh, int nkv, int hd, float scale, void* stream) {
    return cai_flash_attn_bwd_ex(qkv, out, dout, lse, delta, dqkv, B, S, nh, nkv, hd, scale, 7, 0, stream);
}

CAI_API int cai_flash_attn_bwd_parts(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                                     void* dqkv, int B, int S, int nh, int nkv, int hd, float scale, int parts, void* stream) {
    return cai_flash_attn_bwd_ex(qkv, out, dout, lse, delta, dqkv, B, S, nh, nkv, hd, scale, parts, 0, stream);
}

CAI_API int cai_flash_attn_bwd_ex(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                                  void* dqkv, int B, int S, int nh, int nkv, int hd, float scale, int parts, int variant,
                                  void* stream) {
    if (hd != kAttnHD || S % kAttnTile || nkv <= 0 || nh % nkv) {
        set_last_error("flash_attn_bwd: needs head_dim 128, seq %% 128 == 0, heads %% kv_heads == 0");
        return CAI_K_BAD_ARG;
    }
    if (B <= 0 || S <= 0) return CAI_K_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long ld = static_cast<long long>(nh + 2 * nkv) * hd;
    const long long ldo = static_cast<long long>(nh) * hd;
    CUtensorMap tm_qkv, tm_do;
    if (!encode_tmap_2d(&tm_qkv, qkv, static_cast<uint64_t>(B) * S, ld, ld, 64, kAttnTile, 2)) return CAI_K_BAD_ARG;
    if (!encode_tmap_2d(&tm_do, dout, static_cast<uint64_t>(B) * S, ldo, ldo, 64, kAttnTile, 2)) return CAI_K_BAD_ARG;
    const bool pipelined = variant != 1;
    CUtensorMap tm_qkv64, tm_do64;  // 64-row boxes: the half tiles the pipelined kernels stream
    if (pipelined && (!encode_tmap_2d(&tm_qkv64, qkv, static_cast<uint64_t>(B) * S, ld, ld, 64, 64, 2) ||
                      !encode_tmap_2d(&tm_do64, dout, static_cast<uint64_t>(B) * S, ldo, ldo, 64, 64, 2)))
        return CAI_K_BAD_ARG;
    constexpr int smem_bytes = 6 * kAttnTileBytes + 2048 + 1024 + 256;
    static bool configured[64] = {};
    const int dev = current_device();
    if (!configured[dev & 63]) {
        if (cudaFuncSetAttribute(attn_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess ||
            cudaFuncSetAttribute(attn_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess ||
            cudaFuncSetAttribute(attn_dkdv_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess ||
            cudaFuncSetAttribute(attn_dq_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) {
            set_last_error("cudaFuncSetAttribute(attn_bwd) failed");
            return CAI_K_CUDA;
        }
        configured[dev & 63] = true;
    }
    const long long warps = static_cast<long long>(B) * S * nh;
    if (parts & 1)
        attn_delta_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(dout), delta, B, S, nh);
    AttnBwdParams p;
    p.B = B; p.S = S; p.nh = nh; p.nkv = nkv;
    p.scale = scale;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.lse = lse;
    p.delta = delta;
    p.dqkv = static_cast<__nv_bfloat16*>(dqkv);
    p.status = status_words(dev);
    const int nq = S / kAttnTile;
    // Few kv groups per GPU (tensor parallelism): one CTA per query head instead of per kv group shortens the
    // longest CTA by the group size; the heads of a group then add into dK / dV in turn (chain counters).
    p.split_heads = 0;
    p.chain = nullptr;
    const size_t need = static_cast<size_t>(B) * nkv * nq;
    if ((parts & 2) && nh > nkv && static_cast<long long>(nq) * nkv * B < sm_count(dev) &&
        static_cast<long long>(nq) * nh * B <= sm_count(dev) && need <= kAttnChainSlots) {
        // the counters live in a device array of the library: nothing is allocated on this path. The first call
        // on a device resolves the array's address (which may load the module), so it should come before any
        // stream capture; later calls only enqueue work.
        static unsigned int* chain_ptr[64] = {};
        if (!chain_ptr[dev & 63] &&
            cudaGetSymbolAddress(reinterpret_cast<void**>(&chain_ptr[dev & 63]), g_attn_chain) != cudaSuccess) {
            set_last_error("attn_bwd: cannot resolve the chain counters");
            return CAI_K_CUDA;
        }
        if (cudaMemsetAsync(chain_ptr[dev & 63], 0, need * sizeof(unsigned int), st) != cudaSuccess) return CAI_K_CUDA;
        p.split_heads = 1;
        p.chain = chain_ptr[dev & 63];
    }
    const dim3 grid_kv(nq, p.split_heads ? nh : nkv, B), grid_q(nq, nh, B);
    if (pipelined) {
        if (parts & 2) attn_dkdv_pipe_kernel<<<grid_kv, kAttnBwdThreads, smem_bytes, st>>>(tm_qkv, tm_qkv64, tm_do64, p);
        if (parts & 4) attn_dq_pipe_kernel<<<grid_q, kAttnBwdThreads, smem_bytes, st>>>(tm_qkv, tm_do, tm_qkv64, p);
    } else {
        if (parts & 2) attn_dkdv_kernel<<<grid_kv, kAttnBwdThreads, smem_bytes, st>>>(tm_qkv, tm_do, p);
        if (parts & 4) attn_dq_kernel<<<grid_q, kAttnBwdThreads, smem_bytes, st>>>(tm_qkv, tm_do, p);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_error("attn_bwd launch failed: %s", cudaGetErrorString(e));
        return CAI_K_CUDA;
    }
    return CAI_K_OK;
}
