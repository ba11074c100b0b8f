// fused.h - host-side launchers of the fused compute+collective kernels (internal to
// libcai_kernels.so; the executor calls them when it meets the fused op kinds of a plan).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace cai {
struct PeerTable;
struct GatherJob;
void gather_job_finish(GatherJob& job);
}

// Gradient reduce-scatter + scale + sharded AdamW + parameter all-gather, one kernel (rs_adamw.cu).
// local_params: the bf16 parameters are sharded like the optimizer state (ZeRO-3); param_off is then the
// arena offset of the local shard and nothing is pushed to the other members.
int cai_fused_rs_adamw(const cai::PeerTable& pt, unsigned long long grad_off, unsigned long long param_off, float* master,
                       float* m, float* v, long long n_flat, long long n_shard, const float* hyper, float gscale,
                       uint32_t seq, unsigned int* done_counter, int local_params, cudaStream_t st,
                       long long bucket_lo = 0, long long bucket_hi = -1, int max_ctas = 0,   // bucket: the part of the flat space this launch covers
                       int staged = 0, float* gacc = nullptr, int acc_only = 0, int acc_first = 0);   // sharded gradients, see rs_adamw.cu

// All-gather of a row-sharded activation fused into the GEMM that consumes it (gemm_tcgen05.cu).
int cai_fused_ag_gemm(const cai::PeerTable& pt, int group_kind, unsigned long long src_off, long long ld_src, void* a_full,
                      const void* B, void* C, int T, int N, int K, long long ldb, long long ldc, int b_mn,
                      int rows_per_rank, const uint32_t* epoch_base, uint32_t seq, int n_copy, cudaStream_t st,
                      int epi = 0, const void* R = nullptr, long long ldr = 0);   // epi: CAI_EPI_BF16 or a SwiGLU epilogue (R: its second tensor)

// GEMM whose epilogue reduce-scatters the product over the group and adds a residual (gemm_tcgen05.cu).
int cai_fused_gemm_rs(const cai::PeerTable& pt, int group_kind, const void* A, const void* B, unsigned long long stage_off,
                      void* out_local, const void* residual, int T, int N, int K, long long lda, long long ldb,
                      long long ldo, long long ldr, int b_mn, int rows_per_rank, const uint32_t* epoch_base, uint32_t seq,
                      cudaStream_t st);

// Parameter gather of a ZeRO-3 layout (gather.cuh): stand-alone (fsdp_gather.cu) and fused into the
// first GEMM that reads the gathered weights (gemm_tcgen05.cu). The job's slot fields are derived here.
int cai_fsdp_gather(const cai::PeerTable& pt, cai::GatherJob job, const uint32_t* epoch_base, uint32_t seq, cudaStream_t st);
int cai_fused_gather_gemm(const cai::PeerTable& pt, const cai::GatherJob& job, const void* A, const void* B, void* C, const void* R,
                          int M, int N, int K, long long lda, long long ldb, long long ldc, long long ldr, int a_mn, int b_mn,
                          int epi, float alpha, const uint32_t* epoch_base, uint32_t seq, cudaStream_t st);
