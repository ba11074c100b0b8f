// attn_common.cuh - pieces shared by the flash-attention forward and backward kernels:
// tile geometry, the exp2 approximation and the two MMA issue patterns (both operands in shared
// memory K-major; A operand in tensor memory with an MN-major B operand).
#pragma once

#include "sm100.cuh"

namespace cai {

constexpr int kAttnHD = 128;
constexpr int kAttnTile = 128;
constexpr int kAttnTileBytes = kAttnTile * kAttnHD * 2;  // 32 KiB: two 64-column sub-tiles
constexpr int kAttnSub = kAttnTileBytes / 2;
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// S[128,128] = Q[128,hd] * K[128,hd]^T, both operands K-major in two 64-column sub-tiles.
__device__ __forceinline__ void issue_qk(uint32_t d_tmem, uint32_t q_smem, uint32_t k_smem, uint32_t idesc) {
#pragma unroll
    for (int k = 0; k < kAttnHD / 16; ++k) {
        const uint32_t off = (k >> 2) * kAttnSub + (k & 3) * 32;
        umma_f16_ss(d_tmem, umma_smem_desc_sw128(q_smem + off, 0, 1024),
                    umma_smem_desc_sw128(k_smem + off, 0, 1024), idesc, k > 0 ? 1u : 0u);
    }
}
// O[128,hd] (+)= P[128,128](TMEM, bf16 pairs) * V[128,hd]; V is the MN-major B operand.
__device__ __forceinline__ void issue_pv(uint32_t d_tmem, uint32_t p_tmem, uint32_t v_smem, uint32_t idesc,
                                         bool accumulate) {
#pragma unroll
    for (int k = 0; k < kAttnTile / 16; ++k) {
        umma_f16_ts(d_tmem, p_tmem + k * 8, umma_smem_desc_sw128(v_smem + k * 2048, kAttnSub, 1024), idesc,
                    (accumulate || k > 0) ? 1u : 0u);
    }
}

// Half-tile forms: a 64-row operand streamed as two 8 KiB sub-tiles (64 rows x 64 columns each).
constexpr int kAttnHalfSub = 64 * 64 * 2;          // 8 KiB
constexpr int kAttnHalfBytes = 2 * kAttnHalfSub;   // 16 KiB: 64 rows x head_dim

// D[128,64] = A[128,hd] * B[64,hd]^T, both K-major: A in two 16 KiB sub-tiles, B in two 8 KiB sub-tiles.
__device__ __forceinline__ void issue_qk_n64(uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem, uint32_t idesc_n64) {
#pragma unroll
    for (int k = 0; k < kAttnHD / 16; ++k) {
        const uint32_t sub = k >> 2, in = (k & 3) * 32;
        umma_f16_ss(d_tmem, umma_smem_desc_sw128(a_smem + sub * kAttnSub + in, 0, 1024),
                    umma_smem_desc_sw128(b_smem + sub * kAttnHalfSub + in, 0, 1024), idesc_n64, k > 0 ? 1u : 0u);
    }
}
// D[128,hd] (+)= A[128,64](TMEM, bf16 pairs) * B[64,hd] with B MN-major in two 8 KiB sub-tiles. The A operand sits
// in two pieces of 16 columns, 32 columns apart (each piece where one warp group read its 32 fp32 columns from).
__device__ __forceinline__ void issue_pv_k64(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_smem, uint32_t idesc,
                                             bool accumulate) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        umma_f16_ts(d_tmem, a_tmem + (k >> 1) * 32 + (k & 1) * 8,
                    umma_smem_desc_sw128(b_smem + k * 2048, kAttnHalfSub, 1024), idesc, (accumulate || k > 0) ? 1u : 0u);
    }
}

}  // namespace cai
