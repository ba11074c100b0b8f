/* cai_kernels.h - C ABI of the sm_100a kernel library (libcai_kernels.so).
 *
 * Every launcher takes raw device pointers and a CUDA stream handle, enqueues work and returns
 * immediately: 0 on success, a negative code on a host-side failure (cai_last_error() has the
 * text). Device-side waits are bounded; a kernel that gives up records a code in the device's
 * status word, which cai_status_read() returns.
 *
 * Matrices are row-major. bf16 tensors are 2-byte brain floats; "f32" are IEEE floats. */
#ifndef CAI_KERNELS_H
#define CAI_KERNELS_H

#include <stdint.h>

#ifdef __cplusplus
#define CAI_API extern "C" __attribute__((visibility("default")))
#else
#define CAI_API
#endif

/* GEMM epilogues */
enum {
    CAI_EPI_BF16 = 0,          /* C(bf16) = alpha*acc */
    CAI_EPI_F32 = 1,           /* C(f32)  = alpha*acc */
    CAI_EPI_F32_ACCUM = 2,     /* C(f32) += alpha*acc */
    CAI_EPI_BF16_RESIDUAL = 3, /* C(bf16) = alpha*acc + R(bf16); R may alias C */
    /* SwiGLU inside the gate/up projection. B holds [gate rows (F); up rows (F)], N = 2F. An output tile covers
     * BN/2 gate columns and the BN/2 up columns of the same features, so the epilogue writes gate and up to
     * C[:, j] / C[:, F + j] (the layout the backward reads) and act = silu(gate) * up to R[:, j] (bf16, pitch ldr;
     * R is an OUTPUT here). F must be a multiple of 128; B must be stored [N, K]. */
    CAI_EPI_SWIGLU = 4,
    /* SwiGLU backward inside the down projection's input-gradient product (acc = dact, N = F): R is the saved
     * [gate | up] activation (pitch ldr, 2F columns), C receives [dgate | dup] (pitch ldc, 2F columns). */
    CAI_EPI_SWIGLU_BWD = 5
};

CAI_API int cai_status_read(int clear);
/* Time limit (microseconds) of every in-kernel wait on a flag another GPU sets; 0 = default (about 2 s). */
CAI_API int cai_set_wait_limit_us(unsigned int us);
/* Host-side abort: kernels of the current device that sit in a bounded wait give up at once (status 108). */
CAI_API int cai_status_abort(void);
CAI_API const char* cai_last_error(void);
CAI_API int cai_sm_count(void);

/* C[M,N] = alpha * sum_k A(m,k) B(n,k).
 * a_mn_major = 0: A is stored [M,K] (pitch lda); 1: A is stored [K,M].
 * b_mn_major = 0: B is stored [N,K] (pitch ldb); 1: B is stored [K,N].
 * sm_limit > 0 caps the number of CTAs (to leave SMs to a concurrent stream). */
CAI_API int cai_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                          long long lda, long long ldb, long long ldc, long long ldr, int a_mn_major,
                          int b_mn_major, int epi, float alpha, int sm_limit, void* stream);

/* Same product over ragged slabs (expert buffers of a mixture-of-experts layer). The segmented
 * dimension is cut into slabs of seg_rows rows (a multiple of 128); only the first
 * seg_counts[slab] rows of a slab hold data (device array). seg_mode 1: M is segmented, output
 * tiles past a slab's count are neither computed nor written. seg_mode 2: K is segmented (weight
 * gradient), k-blocks past a slab's count are skipped; rows between the count and the next multiple
 * of 64 must be zero in A and B. */
CAI_API int cai_gemm_bf16_seg(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                              long long lda, long long ldb, long long ldc, long long ldr, int a_mn_major,
                              int b_mn_major, int epi, float alpha, const int* seg_counts, int seg_rows, int seg_mode,
                              int sm_limit, void* stream);

/* `groups` independent products of one shape in ONE launch (the local experts of a mixture-of-experts layer):
 * group g reads A and B at row coordinate + g * grp_a / grp_b (rows of the [M,K] or, MN-major, [K,M] tensor),
 * writes C at row + g * grp_c and owns grp_seg entries of seg_counts. MN-major grouped operands need K % 64 == 0. */
CAI_API int cai_gemm_bf16_grouped(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                                  long long ldc, int a_mn_major, int b_mn_major, int epi, const int* seg_counts, int seg_rows,
                                  int seg_mode, int groups, long long grp_a, long long grp_b, long long grp_c, int grp_seg,
                                  void* stream);

/* ---- fused compute + collective GEMMs over peer memory, C forms with explicit member arena bases
 * (bases[rank] is the local one; sig_off: arena offset of the signal block, see cai_signal_block_bytes;
 * epoch_base: device word, epoch of the call = *epoch_base + 2 * seq and must grow from call to call).
 * ag_gemm: C[T,N] = gather_rows(every member's [T/size, K] block at arena offset src_off) * op(B);
 *          a_full [T,K] local receives the gathered rows.
 * gemm_rs: out_local[T/size, N] = residual + sum over members of (A[T,K] * op(B))[my rows]; stage_off is the
 *          arena offset of a [size, T/size, N] bf16 staging buffer on every member. */
CAI_API int cai_fused_ag_gemm_c(void* const* bases, int rank, int size, unsigned long long sig_off, int group_kind,
                                unsigned long long src_off, long long ld_src, void* a_full, const void* B, void* C, int T, int N,
                                int K, long long ldb, long long ldc, int b_mn, const unsigned int* epoch_base, unsigned int seq,
                                int n_copy, void* stream);
CAI_API int cai_fused_gemm_rs_c(void* const* bases, int rank, int size, unsigned long long sig_off, int group_kind, const void* A,
                                const void* B, unsigned long long stage_off, void* out_local, const void* residual, int T, int N,
                                int K, long long lda, long long ldb, long long ldo, long long ldr, int b_mn,
                                const unsigned int* epoch_base, unsigned int seq, void* stream);

/* ---- fp8 (e4m3) GEMM with block scales: C[M,N] = sum_kb sa[m,kb] * sb[n/128,kb] * (Aq[m,kb] . Bq[n,kb]).
 * Aq [M,K], Bq [N,K] e4m3 K-major (K % 128 == 0); sa [M,K/128], sb [ceil(N/128),K/128] fp32.
 * epi: CAI_EPI_BF16, CAI_EPI_F32 or CAI_EPI_BF16_RESIDUAL. No counterpart in the reference. */
CAI_API int cai_gemm_fp8_blockscaled(const void* Aq, const float* sa, const void* Bq, const float* sb, void* C, const void* R,
                                     int M, int N, int K, long long lda, long long ldb, long long ldc, long long ldr, int epi,
                                     void* stream);
/* bf16 [rows,cols] -> e4m3 with one scale per row and 128 columns (scale [rows, cols/128], amax/448). */
CAI_API int cai_quant_rows_1x128(const void* x, long long ldx, void* q, long long ldq, float* scale, int rows, int cols,
                                 void* stream);
/* bf16 [rows,cols] -> e4m3 with one scale per 128x128 block (scale [ceil(rows/128), ceil(cols/128)]); qt / scale_t
 * (optional) receive the transposed tensor [cols,rows] and its scale table. */
CAI_API int cai_quant_blocks_128x128(const void* w, long long ldw, void* q, long long ldq, void* qt, long long ldqt, float* scale,
                                     float* scale_t, int rows, int cols, void* stream);

/* ---- normalisation (reference: src/cuda/cai_kernels.cu:37-77, src/refmodel.c:47-77) */
/* y = x * rsqrt(mean(x^2)+eps) * g ; rstd[row] saved for backward. */
CAI_API int cai_rmsnorm_fwd(const void* x, const void* g, void* y, float* rstd, int rows, int H, float eps,
                            void* stream);
/* dx (+)= rmsnorm backward ; dg_partial is scratch [cai_rmsnorm_bwd_parts(rows), H] f32 ;
 * dg(f32)[H] (+)= sum over rows. */
CAI_API int cai_rmsnorm_bwd_parts(int rows);
CAI_API int cai_rmsnorm_bwd(const void* x, const void* g, const float* rstd, const void* dy, void* dx,
                            float* dg, float* dg_partial, int rows, int H, int dx_accumulate,
                            int dg_accumulate, void* stream);

/* ---- rotary embedding, in place on the q and k heads of a packed [T, (nh+2*nkv)*hd] buffer.
 * table is float2 [seq, hd/2] (cos, sin); position of row t is t % seq. inverse=1 applies the
 * transpose rotation (backward). */
CAI_API int cai_rope_table(float* table, int seq, int hd, float theta, void* stream);
CAI_API int cai_rope_apply(void* qkv, const float* table, int T, int seq, int nh, int nkv, int hd,
                           long long ld, int inverse, void* stream);

/* ---- SwiGLU on a packed [T, 2F] gate|up buffer (reference: src/cuda/cai_kernels.cu:146-160) */
CAI_API int cai_swiglu_fwd(const void* gu, void* act, int T, int F, void* stream);
CAI_API int cai_swiglu_bwd(const void* gu, const void* dact, void* dgu, int T, int F, void* stream);

/* ---- embedding (reference: src/cuda/cai_kernels.cu:19-34). vocab_lo/vocab_hi give the slice of
 * the vocabulary this rank owns; tokens outside produce zeros / are skipped. */
CAI_API int cai_embed_fwd(const int* tokens, const void* E, void* out, int T, int H, int vocab_lo, int vocab_hi,
                          void* stream);
CAI_API int cai_embed_bwd(const int* tokens, const void* dout, float* dE, int T, int H, int vocab_lo,
                          int vocab_hi, void* stream);

/* ---- fused softmax cross-entropy over bf16 logits [rows, V] (pitch ld).
 * In place: logits are overwritten by dlogits = (softmax - onehot) * grad_scale.
 * loss_sum (f32[1]) += sum of row losses * loss_scale. targets < 0 are ignored.
 * (reference: src/cuda/cai_kernels.cu:165-184) */
CAI_API int cai_cross_entropy(void* logits, const int* targets, float* loss_sum, float* row_lse, int rows, int V,
                              long long ld, float grad_scale, float loss_scale, void* stream);

/* Vocabulary-parallel cross-entropy in three steps; the caller max-reduces rowmax and sum-reduces
 * rowsum over the tensor-parallel group in between. vocab_lo is the first vocabulary id of this
 * rank's V columns; add_lse is 1 on exactly one rank of the group so that the summed losses are
 * lse - logit[target]. */
CAI_API int cai_ce_rowmax(const void* logits, float* rowmax, int rows, int V, long long ld, void* stream);
CAI_API int cai_ce_rowsum(const void* logits, const float* rowmax, float* rowsum, int rows, int V, long long ld,
                          void* stream);
CAI_API int cai_ce_grad_tp(void* logits, const int* targets, const float* rowmax, const float* rowsum, float* loss_sum,
                           int rows, int V, long long ld, int vocab_lo, int add_lse, float grad_scale, float loss_scale,
                           void* stream);

/* ---- AdamW on an fp32 master copy with bf16 write-back
 * (reference: src/refmodel.c:481-492, src/cuda/cai_kernels.cu:185-194).
 * p -= lr * (mhat / (sqrt(vhat) + eps) + wd * p); grad is multiplied by grad_scale first. */
CAI_API int cai_adamw(float* master, float* m, float* v, const float* grad, void* param_bf16, long long n,
                      float lr, float beta1, float beta2, float eps, float wd, float grad_scale, int step,
                      void* stream);

/* ---- small utilities */
CAI_API int cai_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream);
CAI_API int cai_cast_bf16_to_f32(const void* src, float* dst, long long n, void* stream);
CAI_API int cai_fill_f32(float* dst, float v, long long n, void* stream);
CAI_API int cai_add_bf16(const void* a, const void* b, void* out, long long n, void* stream);
CAI_API int cai_l2_flush(void* scratch, long long bytes, void* stream);

/* ---- causal GQA flash attention (reference: src/cuda/cai_kernels.cu:80-143)
 * qkv is packed [B*S, (nh+2*nkv)*hd] bf16, head_dim 128. out is [B*S, nh*hd] bf16,
 * lse is f32 [B, nh, S]. */
CAI_API int cai_flash_attn_fwd(const void* qkv, void* out, float* lse, int B, int S, int nh, int nkv, int hd,
                               float scale, void* stream);
/* force_variant: 0 = chosen from the grid size, 1 = one query tile per CTA with the score MMA a block ahead,
 * 2 = two query tiles per CTA in ping-pong. */
CAI_API int cai_flash_attn_fwd_variant(const void* qkv, void* out, float* lse, int B, int S, int nh, int nkv, int hd,
                                       float scale, int force_variant, void* stream);
/* dqkv packed like qkv. delta is scratch f32 [B, nh, S]. */
CAI_API int cai_flash_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                               void* dqkv, int B, int S, int nh, int nkv, int hd, float scale, void* stream);
/* The same in separately launchable parts (bit 0: delta = rowsum(dO * O), bit 1: dK / dV, bit 2: dQ; the last two
 * both need delta and write disjoint columns of dqkv, so they may run on different streams).
 * With few heads (GQA, grid of the dK / dV part no larger than the SM count) the dK / dV part runs one CTA per query
 * head and chains the heads of a kv group through counters in ONE device array of the library, cleared by each
 * call: two calls whose dK / dV parts overlap on the GPU race on it, so issue those from one stream (or order
 * them with events). The first such call on a device resolves the array's address and should precede any stream
 * capture. */
CAI_API int cai_flash_attn_bwd_parts(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                                     void* dqkv, int B, int S, int nh, int nkv, int hd, float scale, int parts, void* stream);
#endif /* CAI_KERNELS_H */
