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
