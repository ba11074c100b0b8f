// flash_attn_fwd.cu - causal grouped-query flash attention forward for sm_100a, head_dim 128.
//
// One CTA owns two adjacent 128-row query tiles (A and B) of one head and sweeps the key/value
// tiles they may attend to. Warp 0 streams Q, K and V tiles with TMA straight out of the packed
// QKV activation; warp 1 issues the tcgen05 MMAs; warps 4-7 and 8-11 are the softmax groups of
// tile A and tile B, one thread per query row. Scores live in tensor memory: S = Q K^T lands in
// TMEM, the softmax group reads it with tcgen05.ld, writes the bf16 probabilities back over the
// same columns with tcgen05.st, and O += P V consumes P directly from TMEM as the A operand.
// While one group runs its softmax the tensor core works on the other tile, so the two overlap.
// The running maximum is only refreshed (and O rescaled in TMEM) when it grew by more than 2^8,
// which keeps that read-modify-write of O rare.
//
// TMEM map (512 columns): S_A/P_A 0-127, S_B/P_B 128-255, O_A 256-383, O_B 384-511.
//
// Replaces the one-thread-per-query kernel of the reference, which materialises the full
// [B, heads, T, T] probability tensor and has no GQA (src/cuda/cai_kernels.cu:80-109).
#include <math.h>

#include "cai_kernels.h"
#include "host_common.h"
#include "attn_common.cuh"
#include "sm100.cuh"

namespace cai {

constexpr int kAttnFwdThreads = 384;

struct AttnFwdParams {
    int B, S, nh, nkv;
    float scale_log2;
    __nv_bfloat16* out;
    float* lse;
    int* status;
};

__global__ void __launch_bounds__(kAttnFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm, const AttnFwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                            // 2 tiles
    uint8_t* sK = smem + 2 * kAttnTileBytes;       // 2 stages
    uint8_t* sV = smem + 4 * kAttnTileBytes;       // 2 stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kAttnTileBytes);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = bars + 3;
    uint64_t* v_full = bars + 5;
    uint64_t* v_empty = bars + 7;
    uint64_t* s_full = bars + 9;
    uint64_t* p_full = bars + 11;
    uint64_t* o_final = bars + 13;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // CTAs are dispatched in linear block order; walk the query tiles slowest so that the heaviest
    // (latest) tiles of every head start first and the light ones fill the tail of the grid. (Pairing
    // tile i with tile last - i balances the CTAs but was slower: a step with one live tile costs as
    // much as a step with two.)
    const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    const int heads_all = gridDim.y * gridDim.z;
    const int pair = gridDim.x - 1 - lin / heads_all;
    const int h = (lin % heads_all) % gridDim.y, b = (lin % heads_all) / gridDim.y;
    const int g = h / (p.nh / p.nkv);
    const int qA = pair * 2 * kAttnTile, qB = qA + kAttnTile;
    const int nA = qA / kAttnTile + 1;
    const int nB = qB < p.S ? qB / kAttnTile + 1 : 0;
    const int n = nB > nA ? nB : nA;
    const int row_base = b * p.S;
    const int col_q = h * kAttnHD, col_k = (p.nh + g) * kAttnHD, col_v = (p.nh + p.nkv + g) * kAttnHD;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm);
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 4);
            mbar_init(&o_final[i], 1);
        }
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

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer
            mbar_expect_tx(q_full, nB ? 2 * kAttnTileBytes : kAttnTileBytes);
            tma_load_2d(sQ, &tm, q_full, col_q, row_base + qA);
            tma_load_2d(sQ + kAttnSub, &tm, q_full, col_q + 64, row_base + qA);
            if (nB) {
                tma_load_2d(sQ + kAttnTileBytes, &tm, q_full, col_q, row_base + qB);
                tma_load_2d(sQ + kAttnTileBytes + kAttnSub, &tm, q_full, col_q + 64, row_base + qB);
            }
            bool ok = true;
            for (int j = 0; j < n && ok; ++j) {
                const int slot = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                const int kv_row = row_base + j * kAttnTile;
                if (!mbar_wait(&k_empty[slot], ph ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                mbar_expect_tx(&k_full[slot], kAttnTileBytes);
                tma_load_2d(sK + slot * kAttnTileBytes, &tm, &k_full[slot], col_k, kv_row);
                tma_load_2d(sK + slot * kAttnTileBytes + kAttnSub, &tm, &k_full[slot], col_k + 64, kv_row);
                if (!mbar_wait(&v_empty[slot], ph ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                mbar_expect_tx(&v_full[slot], kAttnTileBytes);
                tma_load_2d(sV + slot * kAttnTileBytes, &tm, &v_full[slot], col_v, kv_row);
                tma_load_2d(sV + slot * kAttnTileBytes + kAttnSub, &tm, &v_full[slot], col_v + 64, kv_row);
            }
            if (!ok)
                for (int i = 0; i < 32; ++i) __nanosleep(50000);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer
            const uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
            const uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
            const uint32_t sQa = smem_u32(sQ), sQb = smem_u32(sQ + kAttnTileBytes);
            const uint32_t sK0 = smem_u32(sK), sV0 = smem_u32(sV);
            const uint32_t tS[2] = {tmem_base, tmem_base + 128};
            const uint32_t tO[2] = {tmem_base + 256, tmem_base + 384};
            const uint32_t sQx[2] = {sQa, sQb};
            const int nX[2] = {nA, nB};
            bool ok = mbar_wait(q_full, 0, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN) &&
                      mbar_wait(&k_full[0], 0, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN);
            if (ok) {
                tc_fence_after();
                for (int X = 0; X < 2; ++X)
                    if (nX[X] > 0) {
                        issue_qk(tS[X], sQx[X], sK0, idesc_qk);
                        umma_commit(&s_full[X]);
                    }
                umma_commit(&k_empty[0]);
            }
            for (int j = 0; j < n && ok; ++j) {
                const int slot = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                if (!mbar_wait(&v_full[slot], ph, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                const int ns = (j + 1) & 1;
                const uint32_t nph = ((j + 1) >> 1) & 1;
                for (int X = 0; X < 2 && ok; ++X) {
                    if (j >= nX[X]) continue;
                    if (!mbar_wait(&p_full[X], j & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                    tc_fence_after();
                    issue_pv(tO[X], tS[X], sV0 + slot * kAttnTileBytes, idesc_pv, j > 0);
                    if (j + 1 < nX[X]) {
                        if (!mbar_wait(&k_full[ns], nph, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                        tc_fence_after();
                        issue_qk(tS[X], sQx[X], sK0 + ns * kAttnTileBytes, idesc_qk);
                        umma_commit(&s_full[X]);
                    } else {
                        umma_commit(&o_final[X]);
                    }
                }
                if (!ok) break;
                umma_commit(&v_empty[slot]);
                if (j + 1 < n) umma_commit(&k_empty[ns]);
            }
        }
    } else if (warp >= 4) {
        // ---------------- softmax groups: warps 4-7 own tile A, warps 8-11 own tile B
        const int X = warp >= 8 ? 1 : 0;
        const int nx = X ? nB : nA;
        if (nx > 0) {
            const int r = (warp & 3) * 32 + lane;          // row inside the tile == TMEM lane
            const int q0 = X ? qB : qA;
            const uint32_t lane_bits = static_cast<uint32_t>((warp & 3) * 32) << 16;
            const uint32_t tS = tmem_base + X * 128 + lane_bits;
            const uint32_t tO = tmem_base + 256 + X * 128 + lane_bits;
            float m_used = -INFINITY, l = 0.f;
            bool ok = true;
            for (int j = 0; j < nx; ++j) {
                if (!mbar_wait_warp(&s_full[X], j & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                tc_fence_after();
                const bool diag = (j == nx - 1);
                // the whole score row (128 fp32) comes into registers with one wait and is used for both the
                // row maximum and the exponentials
                uint32_t sc[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld_32x32(tS + c * 32, sc[c]);
                tmem_ld_wait();
                float mx = -INFINITY;
                if (!diag) {
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        m0 = fmaxf(m0, __uint_as_float(sc[0][e]));
                        m1 = fmaxf(m1, __uint_as_float(sc[1][e]));
                        m2 = fmaxf(m2, __uint_as_float(sc[2][e]));
                        m3 = fmaxf(m3, __uint_as_float(sc[3][e]));
                    }
                    mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int e = 0; e < 32; ++e)
                            if (c * 32 + e <= r) mx = fmaxf(mx, __uint_as_float(sc[c][e]));
                }
                const float m_new = fmaxf(m_used, mx * p.scale_log2);
                if (__any_sync(0xffffffffu, m_new > m_used + 8.f)) {
                    const float alpha = fast_exp2(m_used - m_new);  // 0 on the first tile
                    l *= alpha;
                    if (j > 0) {
#pragma unroll 1
                        for (int c = 0; c < 4; ++c) {
                            uint32_t v[32];
                            tmem_ld_32x32(tO + c * 32, v);
                            tmem_ld_wait();
#pragma unroll
                            for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                            tmem_st_32x32(tO + c * 32, v);
                        }
                        tmem_st_wait();
                    }
                    m_used = m_new;
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t pk[16];
                    float l0 = 0.f, l1 = 0.f;
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        float p0 = fast_exp2(fmaf(__uint_as_float(sc[c][e]), p.scale_log2, -m_used));
                        float p1 = fast_exp2(fmaf(__uint_as_float(sc[c][e + 1]), p.scale_log2, -m_used));
                        if (diag) {
                            if (c * 32 + e > r) p0 = 0.f;
                            if (c * 32 + e + 1 > r) p1 = 0.f;
                        }
                        l0 += p0;
                        l1 += p1;
                        pk[e >> 1] = pack_bf16(p0, p1);
                    }
                    l += l0 + l1;
                    tmem_st_32x16(tS + c * 16, pk);
                }
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive_warp(&p_full[X]);
            }
            if (ok && mbar_wait_warp(&o_final[X], 0, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) {
                tc_fence_after();
                const float inv = 1.f / l;
                const long long grow = static_cast<long long>(row_base) + q0 + r;
                __nv_bfloat16* orow = p.out + grow * (static_cast<long long>(p.nh) * kAttnHD) + h * kAttnHD;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(tO + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) {
                        uint4 o;
                        o.x = pack_bf16(__uint_as_float(v[j4 * 8 + 0]) * inv, __uint_as_float(v[j4 * 8 + 1]) * inv);
                        o.y = pack_bf16(__uint_as_float(v[j4 * 8 + 2]) * inv, __uint_as_float(v[j4 * 8 + 3]) * inv);
                        o.z = pack_bf16(__uint_as_float(v[j4 * 8 + 4]) * inv, __uint_as_float(v[j4 * 8 + 5]) * inv);
                        o.w = pack_bf16(__uint_as_float(v[j4 * 8 + 6]) * inv, __uint_as_float(v[j4 * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + j4 * 8) = o;
                    }
                }
                if (p.lse)
                    p.lse[(static_cast<long long>(b) * p.nh + h) * p.S + q0 + r] =
                        (m_used + log2f(l)) * 0.6931471805599453f;
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


// ---------------------------------------------------------------------------- one tile per CTA
// Variant for grids that do not fill the GPU (few heads per GPU under tensor parallelism), where the time is
// the critical path of the heaviest CTA. One CTA owns ONE query tile, the scores are double buffered in tensor
// memory and the MMA warp runs one key block ahead: S(j+1) = Q K(j+1)^T is issued before the softmax of block
// j has finished, so a step of the chain costs a softmax, not a softmax plus two MMAs plus two barrier round
// trips. O is rescaled only after the P V of the previous block has completed (own barrier, waited for in
// the rare rescale path, otherwise at the end of the step when it has long completed).
//
// TMEM map: S0/P0 0-127, S1/P1 128-255, O 256-383.
constexpr int kAttnFwd1Threads = 256;

__global__ void __launch_bounds__(kAttnFwd1Threads, 1)
attn_fwd1_kernel(const __grid_constant__ CUtensorMap tm, const AttnFwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = smem + 1 * kAttnTileBytes;       // 2 stages
    uint8_t* sV = smem + 3 * kAttnTileBytes;       // 2 stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 5 * kAttnTileBytes);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = bars + 3;
    uint64_t* v_full = bars + 5;
    uint64_t* v_empty = bars + 7;
    uint64_t* s_full = bars + 9;    // [2] scores of a block are in S[b]
    uint64_t* p_full = bars + 11;   // [2] probabilities of a block are in S[b]
    uint64_t* pv_done = bars + 13;  // P V of a block has completed (O may be touched)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    const int heads_all = gridDim.y * gridDim.z;
    const int tile = gridDim.x - 1 - lin / heads_all;   // heaviest (latest) query tiles of every head first
    const int h = (lin % heads_all) % gridDim.y, b = (lin % heads_all) / gridDim.y;
    const int g = h / (p.nh / p.nkv);
    const int q0 = tile * kAttnTile;
    const int n = tile + 1;                              // key blocks up to the diagonal
    const int row_base = b * p.S;
    const int col_q = h * kAttnHD, col_k = (p.nh + g) * kAttnHD, col_v = (p.nh + p.nkv + g) * kAttnHD;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm);
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 4);
        }
        mbar_init(pv_done, 1);
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

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, kAttnTileBytes);
            tma_load_2d(sQ, &tm, q_full, col_q, row_base + q0);
            tma_load_2d(sQ + kAttnSub, &tm, q_full, col_q + 64, row_base + q0);
            bool ok = true;
            for (int j = 0; j < n && ok; ++j) {
                const int slot = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                const int kv_row = row_base + j * kAttnTile;
                if (!mbar_wait(&k_empty[slot], ph ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                mbar_expect_tx(&k_full[slot], kAttnTileBytes);
                tma_load_2d(sK + slot * kAttnTileBytes, &tm, &k_full[slot], col_k, kv_row);
                tma_load_2d(sK + slot * kAttnTileBytes + kAttnSub, &tm, &k_full[slot], col_k + 64, kv_row);
                if (!mbar_wait(&v_empty[slot], ph ^ 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                mbar_expect_tx(&v_full[slot], kAttnTileBytes);
                tma_load_2d(sV + slot * kAttnTileBytes, &tm, &v_full[slot], col_v, kv_row);
                tma_load_2d(sV + slot * kAttnTileBytes + kAttnSub, &tm, &v_full[slot], col_v + 64, kv_row);
            }
            if (!ok)
                for (int i = 0; i < 32; ++i) __nanosleep(50000);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
            const uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
            const uint32_t sQa = smem_u32(sQ), sK0 = smem_u32(sK), sV0 = smem_u32(sV);
            const uint32_t tS[2] = {tmem_base, tmem_base + 128};
            const uint32_t tO = tmem_base + 256;
            bool ok = mbar_wait(q_full, 0, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN) &&
                      mbar_wait(&k_full[0], 0, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN);
            if (ok) {
                tc_fence_after();
                issue_qk(tS[0], sQa, sK0, idesc_qk);
                umma_commit(&s_full[0]);
                umma_commit(&k_empty[0]);
            }
            for (int j = 0; j < n && ok; ++j) {
                const int slot = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                if (j + 1 < n) {
                    // one block ahead: S[(j+1)&1] last held P(j-1), whose P V was issued before this MMA
                    const int ns = (j + 1) & 1;
                    if (!mbar_wait(&k_full[ns], ((j + 1) >> 1) & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                    tc_fence_after();
                    issue_qk(tS[ns], sQa, sK0 + ns * kAttnTileBytes, idesc_qk);
                    umma_commit(&s_full[ns]);
                    umma_commit(&k_empty[ns]);
                }
                if (!mbar_wait(&p_full[slot], ph, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN) ||
                    !mbar_wait(&v_full[slot], ph, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                tc_fence_after();
                issue_pv(tO, tS[slot], sV0 + slot * kAttnTileBytes, idesc_pv, j > 0);
                umma_commit(&v_empty[slot]);
                umma_commit(pv_done);
            }
        }
    } else if (warp >= 4) {
        const int r = (warp & 3) * 32 + lane;          // row inside the tile == TMEM lane
        const uint32_t lane_bits = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tO = tmem_base + 256 + lane_bits;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n; ++j) {
            const uint32_t tS = tmem_base + (j & 1) * 128 + lane_bits;
            if (!mbar_wait_warp(&s_full[j & 1], (j >> 1) & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
            tc_fence_after();
            const bool diag = (j == n - 1);
            uint32_t sc[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32(tS + c * 32, sc[c]);
            tmem_ld_wait();
            float mx = -INFINITY;
            if (!diag) {
                float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    m0 = fmaxf(m0, __uint_as_float(sc[0][e]));
                    m1 = fmaxf(m1, __uint_as_float(sc[1][e]));
                    m2 = fmaxf(m2, __uint_as_float(sc[2][e]));
                    m3 = fmaxf(m3, __uint_as_float(sc[3][e]));
                }
                mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if (c * 32 + e <= r) mx = fmaxf(mx, __uint_as_float(sc[c][e]));
            }
            const float m_new = fmaxf(m_used, mx * p.scale_log2);
            bool waited_pv = false;
            if (__any_sync(0xffffffffu, m_new > m_used + 8.f)) {
                const float alpha = fast_exp2(m_used - m_new);  // 0 on the first block
                l *= alpha;
                if (j > 0) {
                    // O is complete up to block j-1 only when that block's P V has finished
                    if (!mbar_wait_warp(pv_done, (j - 1) & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
                    waited_pv = true;
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t v[32];
                        tmem_ld_32x32(tO + c * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                        tmem_st_32x32(tO + c * 32, v);
                    }
                    tmem_st_wait();
                }
                m_used = m_new;
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t pk[16];
                float l0 = 0.f, l1 = 0.f;
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float p0 = fast_exp2(fmaf(__uint_as_float(sc[c][e]), p.scale_log2, -m_used));
                    float p1 = fast_exp2(fmaf(__uint_as_float(sc[c][e + 1]), p.scale_log2, -m_used));
                    if (diag) {
                        if (c * 32 + e > r) p0 = 0.f;
                        if (c * 32 + e + 1 > r) p1 = 0.f;
                    }
                    l0 += p0;
                    l1 += p1;
                    pk[e >> 1] = pack_bf16(p0, p1);
                }
                l += l0 + l1;
                tmem_st_32x16(tS + c * 16, pk);
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive_warp(&p_full[j & 1]);
            // every phase of pv_done is consumed exactly once per step, so its parity never runs ahead
            if (j > 0 && !waited_pv &&
                !mbar_wait_warp(pv_done, (j - 1) & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) { ok = false; break; }
        }
        if (ok && mbar_wait_warp(pv_done, (n - 1) & 1, abort_flag, p.status, CAI_DEV_TIMEOUT_ATTN)) {
            tc_fence_after();
            const float inv = 1.f / l;
            const long long grow = static_cast<long long>(row_base) + q0 + r;
            __nv_bfloat16* orow = p.out + grow * (static_cast<long long>(p.nh) * kAttnHD) + h * kAttnHD;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tO + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int j4 = 0; j4 < 4; ++j4) {
                    uint4 o;
                    o.x = pack_bf16(__uint_as_float(v[j4 * 8 + 0]) * inv, __uint_as_float(v[j4 * 8 + 1]) * inv);
                    o.y = pack_bf16(__uint_as_float(v[j4 * 8 + 2]) * inv, __uint_as_float(v[j4 * 8 + 3]) * inv);
                    o.z = pack_bf16(__uint_as_float(v[j4 * 8 + 4]) * inv, __uint_as_float(v[j4 * 8 + 5]) * inv);
                    o.w = pack_bf16(__uint_as_float(v[j4 * 8 + 6]) * inv, __uint_as_float(v[j4 * 8 + 7]) * inv);
                    *reinterpret_cast<uint4*>(orow + c * 32 + j4 * 8) = o;
                }
            }
            if (p.lse)
                p.lse[(static_cast<long long>(b) * p.nh + h) * p.S + q0 + r] = (m_used + log2f(l)) * 0.6931471805599453f;
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

CAI_API int cai_flash_attn_fwd(const void* qkv, void* out, float* lse, int B, int S, int nh, int nkv, int hd,
                               float scale, void* stream) {
    return cai_flash_attn_fwd_variant(qkv, out, lse, B, S, nh, nkv, hd, scale, 0, stream);
}

CAI_API int cai_flash_attn_fwd_variant(const void* qkv, void* out, float* lse, int B, int S, int nh, int nkv, int hd,
                                       float scale, int force_variant, void* stream) {
    if (hd != kAttnHD || S % kAttnTile || nkv <= 0 || nh % nkv) {
        set_last_error("flash_attn_fwd: needs head_dim 128, seq %% 128 == 0, heads %% kv_heads == 0 (hd=%d S=%d)", hd, S);
        return CAI_K_BAD_ARG;
    }
    if (B <= 0 || S <= 0) return CAI_K_OK;
    const long long ld = static_cast<long long>(nh + 2 * nkv) * hd;
    CUtensorMap tm;
    if (!encode_tmap_2d(&tm, qkv, static_cast<uint64_t>(B) * S, ld, ld, 64, kAttnTile, 2)) return CAI_K_BAD_ARG;
    constexpr int smem_bytes = 6 * kAttnTileBytes + 1024 + 256;
    static bool configured[64] = {};
    const int dev = current_device();
    if (!configured[dev & 63]) {
        if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) !=
            cudaSuccess) {
            set_last_error("cudaFuncSetAttribute(attn_fwd) failed");
            return CAI_K_CUDA;
        }
        configured[dev & 63] = true;
    }
    AttnFwdParams p;
    p.B = B; p.S = S; p.nh = nh; p.nkv = nkv;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.lse = lse;
    p.status = status_words(dev);
    // Grids that leave SMs idle (few heads per GPU) are bound by their heaviest CTA: one tile per CTA with the
    // score MMA running a block ahead halves that path. Large grids keep two tiles per CTA in ping-pong.
    const long long pair_ctas = static_cast<long long>((S + 2 * kAttnTile - 1) / (2 * kAttnTile)) * nh * B;
    const bool single = force_variant ? force_variant == 1 : pair_ctas < sm_count(dev);
    if (single) {
        constexpr int smem1 = 5 * kAttnTileBytes + 1024 + 256;
        static bool configured1[64] = {};
        if (!configured1[dev & 63]) {
            if (cudaFuncSetAttribute(attn_fwd1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1) != cudaSuccess) {
                set_last_error("cudaFuncSetAttribute(attn_fwd1) failed");
                return CAI_K_CUDA;
            }
            configured1[dev & 63] = true;
        }
        attn_fwd1_kernel<<<dim3(S / kAttnTile, nh, B), kAttnFwd1Threads, smem1, static_cast<cudaStream_t>(stream)>>>(tm, p);
    } else {
        dim3 grid((S + 2 * kAttnTile - 1) / (2 * kAttnTile), nh, B);
        attn_fwd_kernel<<<grid, kAttnFwdThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(tm, p);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_error("attn_fwd launch failed: %s", cudaGetErrorString(e));
        return CAI_K_CUDA;
    }
    return CAI_K_OK;
}
