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
// Roles per CTA: warp 0 issues TMA, warp 1 issues the MMAs, sixteen warps do the exponentials (four groups of four;
// a warp owns 32 TMEM lanes, a group 32 of the step's 128 score columns). A thread turns 16 fp32 columns at a time
// into 8 packed bf16 columns and writes them over the first half of what it has just read, so the groups never
// touch each other's columns and need no barrier inside a step; the MMA reads its A operand in 8-column pieces,
// 16 columns apart. Every warp arrives once (not every thread) on the barrier that releases the gradient MMAs. The
// softmax scale is applied once to the finished dK / dQ, and only diagonal tiles run the code path with the mask.
// Measured on a B200 (what shaped this layout): the issuing thread runs at most about one MMA ahead of the tensor
// pipe, a barrier wait that is already satisfied still costs it 110-240 cycles because its shared-memory access
// queues behind the operand reads of the MMAs, and 128 x 64 score products run at 58 cycles per MMA against 64 for
// 128 x 128 ones; splitting a step into two 64-column half steps to overlap exponentials and MMAs therefore lost
// to the plain 128-column step with more warps on the exponentials.
//
// Replaces the reference's one-thread-per-query backward, which recomputes dp twice, scatters
// dK/dV with atomicAdd and never zeroes dq/dk/dv (src/cuda/cai_kernels.cu:110-143).
#include <math.h>

#include "attn_common.cuh"
#include "cai_kernels.h"
#include "host_common.h"
#include "sm100.cuh"

namespace cai {

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

// Sixteen compute warps: every scheduler has four of them to hide the TMEM and shared-memory latencies.
constexpr int kAttnGroups = 4;
constexpr int kAttnComputeThreads = kAttnGroups * 128;
constexpr int kAttnBwdThreads = 128 + kAttnComputeThreads;  // warp 0 TMA, warp 1 MMA, warps 4-19 compute

__device__ __forceinline__ void bar_sync_compute() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// One 32-column chunk of a finished fp32 accumulator, times `mul`, to bf16 rows (stored, or added to what is there).
template <bool kAdd>
__device__ __forceinline__ void put_acc_chunk(uint32_t tacc, __nv_bfloat16* dst_row, int c, float mul) {
    uint32_t v[32];
    tmem_ld_32x32(tacc + c * 32, v);
    tmem_ld_wait();
#pragma unroll
    for (int j4 = 0; j4 < 4; ++j4) {
        uint4* dst = reinterpret_cast<uint4*>(dst_row + c * 32 + j4 * 8);
        uint32_t o[4];
        uint4 old = make_uint4(0, 0, 0, 0);
        if constexpr (kAdd) old = *dst;
        const uint32_t ov[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            float a = __uint_as_float(v[j4 * 8 + 2 * t]) * mul, b2 = __uint_as_float(v[j4 * 8 + 2 * t + 1]) * mul;
            if constexpr (kAdd) {
                a += bf16_lo(ov[t]);
                b2 += bf16_hi(ov[t]);
            }
            o[t] = pack_bf16(a, b2);
        }
        *dst = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// dK / dV work of one thread on 16 query columns: S^T / dP^T (dP^T `dp_off` columns behind S^T) -> P^T, dS^T
// (unscaled) as bf16 over the first 8 of the 16 columns read.
template <bool kDiag>
__device__ __forceinline__ void dkdv_pass16(uint32_t tS, uint32_t dp_off, const float* L, const float* D,
                                               float scale_log2, int r, int qb) {
    const uint32_t tdP = tS + dp_off;
    uint32_t sv[16], dp[16], pk[8], dk[8];
    tmem_ld_32x16(tS, sv);
    tmem_ld_32x16(tdP, dp);
    const float4* L4 = reinterpret_cast<const float4*>(L);
    const float4* D4 = reinterpret_cast<const float4*>(D);
    float4 l[4], d[4];
#pragma unroll
    for (int e4 = 0; e4 < 4; ++e4) {
        l[e4] = L4[e4];
        d[e4] = D4[e4];
    }
    tmem_ld_wait();
#pragma unroll
    for (int e4 = 0; e4 < 4; ++e4) {
        const float ls[4] = {l[e4].x, l[e4].y, l[e4].z, l[e4].w}, ds[4] = {d[e4].x, d[e4].y, d[e4].z, d[e4].w};
        float pr[4], dsv[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int e = e4 * 4 + t;
            float pv = fast_exp2(__uint_as_float(sv[e]) * scale_log2 - ls[t]);
            if constexpr (kDiag) {
                if (r > qb + e) pv = 0.f;  // key (row r) may not lie after the query (column)
            }
            pr[t] = pv;
            dsv[t] = pv * (__uint_as_float(dp[e]) - ds[t]);
        }
        pk[e4 * 2] = pack_bf16(pr[0], pr[1]);
        pk[e4 * 2 + 1] = pack_bf16(pr[2], pr[3]);
        dk[e4 * 2] = pack_bf16(dsv[0], dsv[1]);
        dk[e4 * 2 + 1] = pack_bf16(dsv[2], dsv[3]);
    }
    tmem_st_32x8(tS, pk);
    tmem_st_32x8(tdP, dk);
    tmem_st_wait();
}

// dQ work of one thread on 16 key columns: S / dP (dP `dp_off` columns behind S) -> dS (unscaled) as bf16 over the
// first 8 of the 16 dP columns read.
template <bool kDiag>
__device__ __forceinline__ void dq_pass16(uint32_t tS, uint32_t dp_off, float lse2, float dl, float scale_log2, int r,
                                             int kb) {
    const uint32_t tdP = tS + dp_off;
    uint32_t sv[16], dp[16], dk[8];
    tmem_ld_32x16(tS, sv);
    tmem_ld_32x16(tdP, dp);
    tmem_ld_wait();
#pragma unroll
    for (int e = 0; e < 16; e += 2) {
        float p0 = fast_exp2(__uint_as_float(sv[e]) * scale_log2 - lse2);
        float p1 = fast_exp2(__uint_as_float(sv[e + 1]) * scale_log2 - lse2);
        if constexpr (kDiag) {
            if (kb + e > r) p0 = 0.f;
            if (kb + e + 1 > r) p1 = 0.f;
        }
        dk[e >> 1] = pack_bf16(p0 * (__uint_as_float(dp[e]) - dl), p1 * (__uint_as_float(dp[e + 1]) - dl));
    }
    tmem_st_32x8(tdP, dk);
    tmem_st_wait();
}

// D[128,hd] (+)= A[128,128](TMEM, bf16 pairs) * B[128,hd] with B MN-major in two 16 KiB sub-tiles; the A operand sits in
// eight pieces of 8 columns, 16 columns apart.
__device__ __forceinline__ void issue_pv_g8(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_smem, uint32_t idesc,
                                            bool accumulate) {
#pragma unroll
    for (int k = 0; k < kAttnTile / 16; ++k) {
        umma_f16_ts(d_tmem, a_tmem + k * 16, umma_smem_desc_sw128(b_smem + k * 2048, kAttnSub, 1024), idesc,
                    (accumulate || k > 0) ? 1u : 0u);
    }
}

// ---------------------------------------------------------------------------- dK / dV, one 128 x 128 step in flight
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
        mbar_init(pds_ready, kAttnComputeThreads / 32);
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
                issue_pv_g8(tdV, tS, aD + slot * kAttnTileBytes, idesc_mn, it > 0);   // dV += P^T dO
                issue_pv_g8(tdK, tdP, aQ + slot * kAttnTileBytes, idesc_mn, it > 0);  // dK += dS^T Q (unscaled)
                umma_commit(&qdo_empty[slot]);
            }
            if (ok) umma_commit(final_bar);
        }
    } else if (warp >= 4) {
        const int r = (warp & 3) * 32 + lane;  // kv row inside the tile == TMEM lane
        const int grp = (warp - 4) >> 2;       // which 32 of the step's 128 query columns
        const uint32_t lane_bits = static_cast<uint32_t>((warp & 3) * 32) << 16;
        bool ok = true;
        // per-row statistics of the query tile (lse from group 0, delta from group 1), fetched one step ahead
        const float* stat = grp == 0 ? p.lse : p.delta;
        auto stat_at = [&](int it) {
            const int h = h_first + it / per_head;
            const int i = j + it % per_head;
            return stat[(static_cast<long long>(b) * p.nh + h) * p.S + i * kAttnTile + r];
        };
        float stat_next = grp < 2 ? stat_at(0) : 0.f;
        for (int it = 0; it < iters; ++it) {
            const int i = j + it % per_head;
            const int buf = it & 1;
            if (grp == 0) sL[buf * 128 + r] = stat_next * 1.4426950408889634f;
            else if (grp == 1) sD[buf * 128 + r] = stat_next;
            if (grp < 2 && it + 1 < iters) stat_next = stat_at(it + 1);
            bar_sync_compute();
            if (!mbar_wait_warp(sdp_full, it & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                const int qb = grp * 32 + cc * 16;  // first query column of this pass
                const uint32_t t = tS + lane_bits + qb;
                if (i == j) dkdv_pass16<true>(t, 128, sL + buf * 128 + qb, sD + buf * 128 + qb, p.scale_log2, r, qb);
                else dkdv_pass16<false>(t, 128, sL + buf * 128 + qb, sD + buf * 128 + qb, p.scale_log2, r, qb);
            }
            tc_fence_before();
            mbar_arrive_warp(pds_ready);
        }
        if (ok && mbar_wait_warp(final_bar, 0, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) {
            tc_fence_after();
            const long long grow = static_cast<long long>(row_base) + j * kAttnTile + r;
            const long long ld = static_cast<long long>(p.nh + 2 * p.nkv) * kAttnHD;
            // groups 0, 1: dK columns 0-63 / 64-127 (times the softmax scale); groups 2, 3: dV
            const bool is_k = grp < 2;
            __nv_bfloat16* dst = p.dqkv + grow * ld + (is_k ? col_k : col_v);
            const uint32_t tacc = (is_k ? tdK : tdV) + lane_bits;
            const float mul = is_k ? p.scale : 1.f;
            const int c0 = (grp & 1) * 2;
            if (!p.split_heads) {
                put_acc_chunk<false>(tacc, dst, c0, mul);
                put_acc_chunk<false>(tacc, dst, c0 + 1, mul);
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
                    if (turn == 0) {
                        put_acc_chunk<false>(tacc, dst, c0, mul);
                        put_acc_chunk<false>(tacc, dst, c0 + 1, mul);
                    } else {
                        put_acc_chunk<true>(tacc, dst, c0, mul);
                        put_acc_chunk<true>(tacc, dst, c0 + 1, mul);
                    }
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

// ---------------------------------------------------------------------------- dQ, one 128 x 128 step in flight
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
        mbar_init(ds_ready, kAttnComputeThreads / 32);
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
                issue_pv_g8(tdQ, tdP, aK + slot * kAttnTileBytes, idesc_mn, j > 0);  // dQ += dS K (unscaled)
                umma_commit(&kv_empty[slot]);
            }
            if (ok) umma_commit(final_bar);
        }
    } else if (warp >= 4) {
        const int r = (warp & 3) * 32 + lane;  // q row inside the tile
        const int grp = (warp - 4) >> 2;       // which 32 of the step's 128 key columns
        const uint32_t lane_bits = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const long long vec = (static_cast<long long>(b) * p.nh + h) * p.S + i * kAttnTile + r;
        const float lse2 = p.lse[vec] * 1.4426950408889634f;
        const float dl = p.delta[vec];
        bool ok = true;
#pragma unroll 1
        for (int j = 0; j < n; ++j) {
            if (!mbar_wait_warp(sdp_full, j & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                const int kb = grp * 32 + cc * 16;  // first key column of this pass
                const uint32_t t = tS + lane_bits + kb;
                if (j == i) dq_pass16<true>(t, 128, lse2, dl, p.scale_log2, r, kb);
                else dq_pass16<false>(t, 128, lse2, dl, p.scale_log2, r, kb);
            }
            tc_fence_before();
            mbar_arrive_warp(ds_ready);
        }
        if (ok && mbar_wait_warp(final_bar, 0, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) {
            tc_fence_after();
            const long long grow = static_cast<long long>(row_base) + i * kAttnTile + r;
            const long long ld = static_cast<long long>(p.nh + 2 * p.nkv) * kAttnHD;
            put_acc_chunk<false>(tdQ + lane_bits, p.dqkv + grow * ld + col_q, grp, p.scale);
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
    return cai_flash_attn_bwd_parts(qkv, out, dout, lse, delta, dqkv, B, S, nh, nkv, hd, scale, 7, stream);
}

CAI_API int cai_flash_attn_bwd_parts(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                                     void* dqkv, int B, int S, int nh, int nkv, int hd, float scale, int parts, void* stream) {
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
    constexpr int smem_bytes = 6 * kAttnTileBytes + 2048 + 1024 + 256;
    static bool configured[64] = {};
    const int dev = current_device();
    if (!configured[dev & 63]) {
        if (cudaFuncSetAttribute(attn_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess ||
            cudaFuncSetAttribute(attn_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) {
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
    if (parts & 2) attn_dkdv_kernel<<<grid_kv, kAttnBwdThreads, smem_bytes, st>>>(tm_qkv, tm_do, p);
    if (parts & 4) attn_dq_kernel<<<grid_q, kAttnBwdThreads, smem_bytes, st>>>(tm_qkv, tm_do, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_error("attn_bwd launch failed: %s", cudaGetErrorString(e));
        return CAI_K_CUDA;
    }
    return CAI_K_OK;
}
