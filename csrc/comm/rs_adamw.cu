// rs_adamw.cu - ONE kernel for the data-parallel end of a step: gradient reduce-scatter, the
// 1/dp (and gradient-accumulation) scale, the sharded AdamW update on the fp32 master copy, and
// the all-gather of the updated bf16 parameters.
//
// Every rank owns a contiguous 1/dp shard of the flat parameter space (master, m, v live only
// there). A launch covers a bucket [lo, hi) of the flat space - the whole space, or one layer's
// parameters, launched on the data-parallel stream as soon as the last microbatch's weight gradients of
// that layer exist, so that the reduction and the update overlap the rest of the backward pass (the
// reference plan places a REDUCE_SCATTER per layer on comm_dp for the same reason,
// src/model.c:501-503). Each rank handles the part of the bucket that falls into its shard (possibly
// nothing: it still takes part in the handshakes, which is how the owners learn that its gradients
// are complete). For each of its elements the owner pulls the fp32 gradient of every replica with
// peer loads over NVLink, sums in registers, applies AdamW, and pushes the new bf16 value into the
// parameter buffer of every replica with peer stores. Nothing is staged, nothing goes through
// NCCL. Cross-GPU ordering: an entry handshake ("my gradients are complete") before the first
// peer load and an exit handshake ("I am done with your memory") before the kernel retires, both
// epoch counters in the signal block (peer.cuh).
//
// Replaces the reference's whole-vector ncclAllReduce after backward followed by a replicated
// AdamW (src/cuda/cai_gpu_train.cu:267-269, src/cuda/cai_nccl.cu:75-80), and is what the plan's
// REDUCE_SCATTER + barrier + OPTIMIZER sequence (src/model.c:501-503,706-711) turns into.
#include <cuda_bf16.h>

#include "../kernels/host_common.h"
#include "../plan/formats.h"
#include "fused.h"
#include "peer.cuh"

namespace cai {

struct RsAdamwParams {
    unsigned long long grad_off, param_off;  // arena offsets, valid on every member
    float* master;
    float* m;
    float* v;
    long long n_flat, n_shard;
    long long bucket_lo, bucket_hi;          // this launch covers [bucket_lo, bucket_hi) of the flat space
    const float* hyper;  // lr, b1, b2, eps, wd, bc1, bc2, [7] = epoch base (uint32 bits)
    float gscale;
    uint32_t seq;
    unsigned int* done_counter;
    int local_params;  // bf16 parameters sharded like the optimizer state: write my shard only
    // Sharded gradients (ZeRO-3 with per-layer buckets): the members' gradients of the bucket sit in a staging buffer
    // (element i of the flat space at grad_off + (i - bucket_lo) * 4) and hold ONE microbatch; the owner keeps the
    // running sum of its elements in `gacc` (indexed like master). acc_only: reduce into gacc and stop (not the last
    // microbatch); acc_first: gacc holds nothing yet.
    int staged;
    float* gacc;
    int acc_only, acc_first;
    int* status;
};

__global__ void __launch_bounds__(256) rs_adamw_kernel(const PeerTable pt, const RsAdamwParams p) {
    __shared__ int ok_s;
    const uint32_t epoch = reinterpret_cast<const uint32_t*>(p.hyper)[7] + 2 * p.seq;
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0) signal_all(pt, GROUP_DP, kSigEntry + pt.rank, epoch);
        ok_s = wait_all(pt, GROUP_DP, kSigEntry, epoch, p.status) ? 1 : 0;
    }
    __syncthreads();
    const bool ok = ok_s != 0;
    if (ok) {
        const float lr = p.hyper[0], b1 = p.hyper[1], b2 = p.hyper[2], eps = p.hyper[3], wd = p.hyper[4],
                    bc1 = p.hyper[5], bc2 = p.hyper[6];
        const long long lo = static_cast<long long>(pt.rank) * p.n_shard;   // my shard: [lo, shard_hi)
        const long long shard_hi = lo + p.n_shard < p.n_flat ? lo + p.n_shard : p.n_flat;
        const long long first = lo > p.bucket_lo ? lo : p.bucket_lo;         // my part of this bucket
        const long long hi = shard_hi < p.bucket_hi ? shard_hi : p.bucket_hi;
        const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
        for (long long i = first + (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < hi; i += stride) {
            float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
            const long long gi = p.staged ? i - p.bucket_lo : i;
#pragma unroll
            for (int mbr = 0; mbr < kMaxPeers; ++mbr) {
                if (mbr < pt.size) {
                    const float4 t = *reinterpret_cast<const float4*>(pt.base[mbr] + p.grad_off + gi * 4);
                    g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
                }
            }
            const long long j = i - lo;
            if (p.gacc) {
                if (!p.acc_first) {
                    const float4 a = *reinterpret_cast<const float4*>(p.gacc + j);
                    g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
                }
                if (p.acc_only) {
                    *reinterpret_cast<float4*>(p.gacc + j) = g;
                    continue;
                }
            }
            const float4 p4 = *reinterpret_cast<const float4*>(p.master + j);
            const float4 m4 = *reinterpret_cast<const float4*>(p.m + j);
            const float4 v4 = *reinterpret_cast<const float4*>(p.v + j);
            float w[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
            const float gg[4] = {g.x * p.gscale, g.y * p.gscale, g.z * p.gscale, g.w * p.gscale};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                mm[e] = b1 * mm[e] + (1.f - b1) * gg[e];
                vv[e] = b2 * vv[e] + (1.f - b2) * gg[e] * gg[e];
                w[e] -= lr * ((mm[e] / bc1) / (sqrtf(vv[e] / bc2) + eps) + wd * w[e]);
            }
            *reinterpret_cast<float4*>(p.master + j) = make_float4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<float4*>(p.m + j) = make_float4(mm[0], mm[1], mm[2], mm[3]);
            *reinterpret_cast<float4*>(p.v + j) = make_float4(vv[0], vv[1], vv[2], vv[3]);
            uint2 o;
            o.x = pack_bf16(w[0], w[1]);
            o.y = pack_bf16(w[2], w[3]);
            if (p.local_params) {
                *reinterpret_cast<uint2*>(pt.base[pt.rank] + p.param_off + j * 2) = o;
            } else {
#pragma unroll
                for (int mbr = 0; mbr < kMaxPeers; ++mbr)
                    if (mbr < pt.size) *reinterpret_cast<uint2*>(pt.base[mbr] + p.param_off + i * 2) = o;
            }
        }
    }
    // Exit handshake by the last CTA of the grid: peers may reuse their gradient buffers and may
    // read their parameters only after every owner has finished with them.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int ticket = atomicAdd(p.done_counter, 1u);
        if (ticket == gridDim.x - 1) {
            *p.done_counter = 0;
            __threadfence();
            if (ok) {
                signal_all(pt, GROUP_DP, kSigExit + pt.rank, epoch + 1);
                wait_all(pt, GROUP_DP, kSigExit, epoch + 1, p.status);
            }
        }
    }
}

}  // namespace cai

using namespace cai;

int cai_fused_rs_adamw(const PeerTable& pt, unsigned long long grad_off, unsigned long long param_off, float* master,
                       float* m, float* v, long long n_flat, long long n_shard, const float* hyper, float gscale,
                       uint32_t seq, unsigned int* done_counter, int local_params, cudaStream_t st,
                       long long bucket_lo, long long bucket_hi, int max_ctas, int staged, float* gacc, int acc_only, int acc_first) {
    if (bucket_hi < 0) bucket_hi = n_flat;
    if ((n_shard & 3) || (n_flat & 3) || (bucket_lo & 3) || (bucket_hi & 3) || bucket_lo < 0 || bucket_lo > bucket_hi || bucket_hi > n_flat) {
        set_last_error("rs_adamw: element counts and bucket bounds must be multiples of 4 (bucket %lld..%lld of %lld)", bucket_lo,
                       bucket_hi, n_flat);
        return CAI_K_BAD_ARG;
    }
    RsAdamwParams p;
    p.grad_off = grad_off; p.param_off = param_off;
    p.master = master; p.m = m; p.v = v;
    p.n_flat = n_flat; p.n_shard = n_shard;
    p.bucket_lo = bucket_lo; p.bucket_hi = bucket_hi;
    p.hyper = hyper; p.gscale = gscale; p.seq = seq;
    p.done_counter = done_counter;
    p.local_params = local_params;
    p.staged = staged; p.gacc = gacc; p.acc_only = acc_only; p.acc_first = acc_first;
    const int dev = current_device();
    p.status = status_words(dev);
    // a bucket that runs beside the backward pass takes a slice of the GPU (max_ctas), the end-of-step launch all of it
    int grid = sm_count(dev) * 4;
    if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
    rs_adamw_kernel<<<grid, 256, 0, st>>>(pt, p);
    if (cudaGetLastError() != cudaSuccess) {
        set_last_error("rs_adamw launch failed");
        return CAI_K_CUDA;
    }
    return 0;
}

// C form with explicit member bases (tests, micro-benchmarks). hyper: 8 device floats (lr, beta1, beta2, eps,
// weight decay, bias corrections 1 and 2, and the epoch base as uint32 bits); scratch: a zeroed device uint32.
extern "C" __attribute__((visibility("default"))) int cai_fused_rs_adamw_c(
    void* const* bases, int rank, int size, unsigned long long sig_off, unsigned long long grad_off, unsigned long long param_off,
    float* master, float* m, float* v, long long n_flat, long long n_shard, const float* hyper, float gscale, unsigned int seq,
    unsigned int* scratch, int local_params, void* stream) {
    if (size < 1 || size > kMaxPeers) return CAI_K_BAD_ARG;
    PeerTable pt{};
    for (int i = 0; i < size; ++i) pt.base[i] = static_cast<uint8_t*>(bases[i]);
    pt.rank = rank;
    pt.size = size;
    pt.sig_off = sig_off;
    return cai_fused_rs_adamw(pt, grad_off, param_off, master, m, v, n_flat, n_shard, hyper, gscale, seq, scratch, local_params,
                              static_cast<cudaStream_t>(stream), 0, -1, 0, 0, nullptr, 0, 0);
}
