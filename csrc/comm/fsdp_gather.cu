// fsdp_gather.cu - stand-alone form of the parameter gather (gather.cuh): stages a range of the
// sharded flat parameter space into a local buffer with TMA bulk copies over NVLink. Used for
// parameters whose first consumer is not a GEMM (embedding rows, the final norm gain); layer
// weights are gathered by the copy CTAs of the first GEMM that reads them (gemm_tcgen05.cu).
//
// The reference has no counterpart on the device (src/model.c:442-451 prices an ALL_GATHER).
#include "../kernels/host_common.h"
#include "../plan/formats.h"
#include "fused.h"
#include "gather.cuh"

namespace cai {

__global__ void __launch_bounds__(32) fsdp_gather_kernel(const PeerTable pt, const GatherJob job, const uint32_t* epoch_base,
                                                         uint32_t seq, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring + kGatherRingBytes);
    if (threadIdx.x == 0) gather_copy_role(pt, job, static_cast<int>(blockIdx.x), *epoch_base + 2 * seq, ring, bars, status);
}

// Fills the derived fields of a job: progress slots of a whole number of copy pieces, at most kSigLocalSlots of them.
void gather_job_finish(GatherJob& job) {
    const long long n = job.hi - job.lo;
    const long long piece = kGatherPiece / 2;
    long long per = (n + kSigLocalSlots - 1) / kSigLocalSlots;
    per = (per + piece - 1) / piece * piece;
    if (per < 4 * piece) per = 4 * piece;
    job.slot_elems = per;
    job.nslots = static_cast<int>((n + per - 1) / per);
}

}  // namespace cai

using namespace cai;

int cai_fsdp_gather(const PeerTable& pt, GatherJob job, const uint32_t* epoch_base, uint32_t seq, cudaStream_t st) {
    if (job.hi <= job.lo || ((job.lo | job.hi | job.n_shard) & 7) || job.n_copy < 1) {
        set_last_error("fsdp_gather: range and shard size must be multiples of 8 elements");
        return CAI_K_BAD_ARG;
    }
    gather_job_finish(job);
    constexpr int smem_bytes = kGatherRingBytes + 128 + 128;
    static bool configured[64] = {};
    const int dev = current_device();
    if (!configured[dev & 63]) {
        if (cudaFuncSetAttribute(fsdp_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) {
            set_last_error("cudaFuncSetAttribute(fsdp_gather) failed");
            return CAI_K_CUDA;
        }
        configured[dev & 63] = true;
    }
    fsdp_gather_kernel<<<job.n_copy, 32, smem_bytes, st>>>(pt, job, epoch_base, seq, status_words(dev));
    return cudaGetLastError() == cudaSuccess ? 0 : CAI_K_CUDA;
}

// C forms with explicit member bases (tests, micro-benchmarks): the stand-alone gather and the GEMM whose copy
// CTAs gather the range that holds its B operand (B = dst + b_elem_off).
static PeerTable fsdp_table_of(void* const* bases, int rank, int size, unsigned long long sig_off) {
    PeerTable pt{};
    for (int i = 0; i < size && i < kMaxPeers; ++i) pt.base[i] = static_cast<uint8_t*>(bases[i]);
    pt.rank = rank;
    pt.size = size;
    pt.sig_off = sig_off;
    return pt;
}
static GatherJob fsdp_job_of(unsigned long long shard_off, long long n_shard, long long lo, long long hi, void* dst, int reverse,
                             int n_copy) {
    GatherJob job{};
    job.shard_off = shard_off; job.n_shard = n_shard; job.lo = lo; job.hi = hi;
    job.dst = static_cast<__nv_bfloat16*>(dst);
    job.reverse = reverse; job.n_copy = n_copy; job.group_kind = GROUP_DP;
    return job;
}
extern "C" __attribute__((visibility("default"))) int cai_fsdp_gather_c(
    void* const* bases, int rank, int size, unsigned long long sig_off, unsigned long long shard_off, long long n_shard,
    long long lo, long long hi, void* dst, int reverse, int n_copy, const unsigned int* epoch_base, unsigned int seq, void* stream) {
    if (size < 1 || size > kMaxPeers) return CAI_K_BAD_ARG;
    return cai_fsdp_gather(fsdp_table_of(bases, rank, size, sig_off), fsdp_job_of(shard_off, n_shard, lo, hi, dst, reverse, n_copy),
                           epoch_base, seq, static_cast<cudaStream_t>(stream));
}
extern "C" __attribute__((visibility("default"))) int cai_fused_gather_gemm_c(
    void* const* bases, int rank, int size, unsigned long long sig_off, unsigned long long shard_off, long long n_shard,
    long long lo, long long hi, void* dst, int reverse, int n_copy, const void* A, long long b_elem_off, void* C, int M, int N,
    int K, long long lda, long long ldb, long long ldc, int b_mn, const unsigned int* epoch_base, unsigned int seq, void* stream) {
    if (size < 1 || size > kMaxPeers) return CAI_K_BAD_ARG;
    const GatherJob job = fsdp_job_of(shard_off, n_shard, lo, hi, dst, reverse, n_copy);
    return cai_fused_gather_gemm(fsdp_table_of(bases, rank, size, sig_off), job, A, job.dst + b_elem_off, C, nullptr, M, N, K, lda,
                                 ldb, ldc, 0, 0, b_mn, CAI_EPI_BF16, 1.0f, epoch_base, seq, static_cast<cudaStream_t>(stream));
}
