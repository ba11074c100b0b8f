// executor.cu - the device runtime: replays a version-2 plan on six CUDA streams.
//
// This is the real-GPU counterpart of the reference's replay loop (src/runtime.c:145-181) and of
// the backend its src/backend_cuda.c:13-30 only sketches: every non-event op becomes a kernel
// launch (or an NCCL call) on the CUDA stream of its logical stream, EVENT_RECORD / EVENT_WAIT
// become cudaEventRecord / cudaStreamWaitEvent on a pre-created pool, and all operands are
// offsets into ONE arena allocation. The host never allocates or synchronises inside a step. A
// whole step can be captured once into a CUDA graph and relaunched, with the per-step scalars
// (learning rate, Adam bias corrections) read from a small device buffer that is refreshed
// before each launch.
//
// NCCL is reached through dlopen so the library has no link-time dependency on it; communicators
// are built from unique ids the launcher distributes (the reference exchanges them through files
// in /tmp, src/cuda/cai_nccl.cu:35-52).
#include <cuda_bf16.h>
#include <dlfcn.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "../comm/fused.h"
#include "../comm/gather.cuh"
#include "../comm/moe.h"
#include "../comm/peer.cuh"
#include "../kernels/cai_kernels.h"
#include "../kernels/host_common.h"
#include "../plan/formats.h"
#include "cai_runtime.h"

namespace cai {

// ------------------------------------------------------------------ NCCL through dlopen
struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, NcclId, int) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*ReduceScatter)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*Send)(const void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*Recv)(void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};
static NcclApi g_nccl;

static bool nccl_load(const char* path) {
    if (g_nccl.handle) return true;
    void* h = dlopen(path && *path ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        set_last_error("dlopen(%s) failed: %s", path ? path : "libnccl.so.2", dlerror());
        return false;
    }
#define LOADSYM(field, name)                                             \
    *reinterpret_cast<void**>(&g_nccl.field) = dlsym(h, name);           \
    if (!g_nccl.field) {                                                 \
        set_last_error("NCCL symbol %s missing", name);                 \
        return false;                                                    \
    }
    LOADSYM(GetUniqueId, "ncclGetUniqueId")
    LOADSYM(CommInitRank, "ncclCommInitRank")
    LOADSYM(CommDestroy, "ncclCommDestroy")
    LOADSYM(AllReduce, "ncclAllReduce")
    LOADSYM(ReduceScatter, "ncclReduceScatter")
    LOADSYM(AllGather, "ncclAllGather")
    LOADSYM(Send, "ncclSend")
    LOADSYM(Recv, "ncclRecv")
    LOADSYM(GroupStart, "ncclGroupStart")
    LOADSYM(GroupEnd, "ncclGroupEnd")
    LOADSYM(GetErrorString, "ncclGetErrorString")
#undef LOADSYM
    g_nccl.handle = h;
    return true;
}

static int nccl_dtype(int dt) {
    switch (dt) {
        case DT_FP32: return 7;
        case DT_BF16: return 9;
        case DT_FP16: return 6;
        case DT_INT32: return 2;
        default: return 1;  // bytes
    }
}

__global__ void adamw_dev_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                 const float* __restrict__ grad, __nv_bfloat16* __restrict__ param, long long n,
                                 const float* __restrict__ hyper, float gscale) {
    // hyper: lr, beta1, beta2, eps, wd, 1-beta1^t, 1-beta2^t
    const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4], bc1 = hyper[5], bc2 = hyper[6];
    const long long i4 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i4 >= n) return;
    const float4 p4 = *reinterpret_cast<const float4*>(master + i4);
    const float4 m4 = *reinterpret_cast<const float4*>(m + i4);
    const float4 v4 = *reinterpret_cast<const float4*>(v + i4);
    const float4 g4 = *reinterpret_cast<const float4*>(grad + i4);
    float p[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
    const float g[4] = {g4.x * gscale, g4.y * gscale, g4.z * gscale, g4.w * gscale};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        mm[e] = b1 * mm[e] + (1.f - b1) * g[e];
        vv[e] = b2 * vv[e] + (1.f - b2) * g[e] * g[e];
        p[e] -= lr * ((mm[e] / bc1) / (sqrtf(vv[e] / bc2) + eps) + wd * p[e]);
    }
    *reinterpret_cast<float4*>(master + i4) = make_float4(p[0], p[1], p[2], p[3]);
    *reinterpret_cast<float4*>(m + i4) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(v + i4) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    __nv_bfloat162 lo = __floats2bfloat162_rn(p[0], p[1]), hi = __floats2bfloat162_rn(p[2], p[3]);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(param + i4) = o;
}

struct Comm {
    void* comm = nullptr;   // forward / only communicator
    void* comm2 = nullptr;  // second communicator of the pipeline group (gradient direction)
    int rank = 0, size = 1;
};

struct TraceRec { uint32_t op; cudaEvent_t start, stop; };

}  // namespace cai

using namespace cai;

struct cai_exec {
    PlanHeader hdr{};
    ExecHeader xhdr{};
    TrainSpec train{};
    ModelSpec model{};
    std::vector<TensorDesc> tensors;
    std::vector<CommGroup> groups;
    std::vector<Op> ops;
    std::vector<ExecOp> exec;
    std::vector<NamedTensor> named;
    std::vector<uint32_t> shapes;
    uint8_t* arena = nullptr;
    int device = 0;
    cudaStream_t streams[ST_COUNT] = {};
    bool owns_stream[ST_COUNT] = {};
    std::vector<cudaEvent_t> events;
    cudaEvent_t fork_ev = nullptr, join_ev[ST_COUNT] = {};
    Comm comms[GROUP_COUNT];
    PeerTable peers[GROUP_COUNT] = {};
    bool has_peers[GROUP_COUNT] = {};
    unsigned int* counters_dev = nullptr;  // scratch words for grid-completion tickets
    uint32_t epochs_per_step = 2;
    int ag_copy_ctas = 0;   // 0: chosen per launch from the GEMM's tile count
    float* hyper_dev = nullptr;   // 8 floats
    // Pinned staging of the per-step scalars. A pinned host-to-device copy reads host memory when it executes,
    // not when it is enqueued, so a caller that enqueues several steps without synchronising must not find
    // the words of step N overwritten by step N+1: a ring of slots, each reused only after the copy that read
    // it has completed (its event), keeps every enqueued step's scalars intact.
    static constexpr int kHyperSlots = 16;
    float* hyper_host = nullptr;  // pinned, kHyperSlots x 8 floats
    cudaEvent_t hyper_ev[kHyperSlots] = {};
    bool hyper_used[kHyperSlots] = {};
    unsigned hyper_next = 0;
    cudaGraphExec_t graph = nullptr;
    bool use_graph = false;
    bool trace_on = false;
    bool nvtx_on = false;   // one NVTX range per op, named by kernel (for timeline tools)
    bool debug_bounds = false;   // check every operand's extent against the plan's tensor table before each launch
    std::vector<TraceRec> trace;
    cai_fused_hook_t fused_hook = nullptr;
    void* fused_ctx = nullptr;
    int sm_limit_hi = 0;
    uint64_t launches = 0;  // kernels / collectives enqueued by the last replay
    // ZeRO-3: a parameter gather waiting to be merged into the GEMM that follows it in the op table
    GatherJob pending_gather{};
    uint32_t pending_seq = 0;
    bool has_pending_gather = false;
    long long n_shard = 0;  // elements of the flat parameter space each data-parallel member owns
    long long n_rep = 0;    // elements of the flat space that are replicated over the data-parallel group
    int flat_ids[5] = {-1, -1, -1, -1, -1};  // tensor ids of @flat_grad, @flat_param, @flat_master, @flat_m, @flat_v

    void* ptr(int t) const { return t >= 0 ? arena + tensors[t].offset : nullptr; }
    long long ld(int t) const { return shapes[static_cast<size_t>(t) * 4 + 2]; }
};

namespace {

int run_op(cai_exec* ex, const Op& op, const ExecOp& x, cudaStream_t st) {
    auto P = [&](int i) { return ex->ptr(x.t[i]); };
    switch (x.kernel) {
        case K_EMBED_FWD:
            return cai_embed_fwd((const int*)P(0), P(1), P(2), x.i[0], x.i[1], x.i[2], x.i[3], st);
        case K_EMBED_BWD:
            return cai_embed_bwd((const int*)P(0), P(1), (float*)P(2), x.i[0], x.i[1], x.i[2], x.i[3], st);
        case K_RMSNORM_FWD:
            return cai_rmsnorm_fwd(P(0), P(1), P(2), (float*)P(3), x.i[0], x.i[1], x.f[0], st);
        case K_RMSNORM_BWD:
            return cai_rmsnorm_bwd(P(0), P(1), (const float*)P(2), P(3), P(4), (float*)P(5), (float*)P(6), x.i[0], x.i[1],
                                   x.i[2], x.i[3], st);
        case K_GEMM: {
            const int ta = x.flags & 1, tb = (x.flags >> 1) & 1, epi = (x.flags >> 4) & 0xF;
            if (ex->has_pending_gather) {
                // the layer's weights are staged by the copy CTAs of this GEMM (B lies in the staged range)
                ex->has_pending_gather = false;
                return cai_fused_gather_gemm(ex->peers[GROUP_DP], ex->pending_gather, P(0), P(1), P(2), P(3), x.i[0], x.i[1], x.i[2],
                                             ex->ld(x.t[0]), ex->ld(x.t[1]), ex->ld(x.t[2]), x.t[3] >= 0 ? ex->ld(x.t[3]) : 0, ta, tb, epi,
                                             x.f[0], reinterpret_cast<const uint32_t*>(ex->hyper_dev) + 7, ex->pending_seq, st);
            }
            if (x.flags & 0x100) {
                // every local expert in one launch: group offsets follow from the operand forms
                const int M = x.i[0], N = x.i[1], K = x.i[2], seg_rows = x.i[3], seg_mode = x.i[4] & 0xFF, groups = x.i[4] >> 8;
                const int epi8 = (x.flags >> 4) & 0xF;
                const long long ga = ta ? K : M, gb = tb ? K : N, gc = M;
                return cai_gemm_bf16_grouped(P(0), P(1), P(2), M, N, K, ex->ld(x.t[0]), ex->ld(x.t[1]), ex->ld(x.t[2]), ta, tb, epi8,
                                             (const int*)P(4), seg_rows, seg_mode, groups, ga, gb, gc,
                                             (seg_mode == 2 ? K : M) / seg_rows, st);
            }
            if (x.t[4] >= 0)  // ragged expert slab: live rows per sub-slab come from a device table
                return cai_gemm_bf16_seg(P(0), P(1), P(2), P(3), x.i[0], x.i[1], x.i[2], ex->ld(x.t[0]), ex->ld(x.t[1]),
                                         ex->ld(x.t[2]), x.t[3] >= 0 ? ex->ld(x.t[3]) : 0, ta, tb, epi, x.f[0],
                                         (const int*)P(4), x.i[3], x.i[4], ex->sm_limit_hi, st);
            return cai_gemm_bf16(P(0), P(1), P(2), P(3), x.i[0], x.i[1], x.i[2], ex->ld(x.t[0]), ex->ld(x.t[1]),
                                 ex->ld(x.t[2]), x.t[3] >= 0 ? ex->ld(x.t[3]) : 0, ta, tb, epi, x.f[0], ex->sm_limit_hi, st);
        }
        case K_ROPE:
            return cai_rope_apply(P(0), (const float*)P(1), x.i[0], x.i[1], x.i[2], x.i[3], x.i[4], ex->ld(x.t[0]),
                                  x.flags & 1, st);
        case K_ATTN_FWD:
            return cai_flash_attn_fwd(P(0), P(1), (float*)P(2), x.i[0], x.i[1], x.i[2], x.i[3], x.i[4], x.f[0], st);
        case K_ATTN_BWD:
            // flags: 0 = the whole backward, otherwise a mask of its parts (1 delta, 2 dK/dV, 4 dQ)
            return cai_flash_attn_bwd_parts(P(0), P(1), P(2), (const float*)P(3), (float*)P(4), P(5), x.i[0], x.i[1], x.i[2],
                                            x.i[3], x.i[4], x.f[0], x.flags ? x.flags : 7, st);
        case K_SWIGLU_FWD: return cai_swiglu_fwd(P(0), P(1), x.i[0], x.i[1], st);
        case K_SWIGLU_BWD: return cai_swiglu_bwd(P(0), P(1), P(2), x.i[0], x.i[1], st);
        case K_CROSS_ENTROPY:
            return cai_cross_entropy(P(0), (const int*)P(1), (float*)P(2), nullptr, x.i[0], x.i[1], ex->ld(x.t[0]), x.f[0],
                                     x.f[1], st);
        case K_CROSS_ENTROPY_TP: {
            // vocabulary-parallel: row max and exp-sum are reduced over the TP group in stream order,
            // on the group's second communicator (the first one belongs to the comm_tp stream)
            const Comm& c = ex->comms[GROUP_TP];
            void* comm = c.comm2 ? c.comm2 : c.comm;
            if (!comm) {
                set_last_error("vocabulary-parallel cross-entropy needs the TP communicator");
                return CAI_K_BAD_ARG;
            }
            float* rowmax = (float*)P(3);
            float* rowsum = rowmax + ex->shapes[static_cast<size_t>(x.t[3]) * 4 + 2];
            const int rows = x.i[0], V = x.i[1];
            int rc = cai_ce_rowmax(P(0), rowmax, rows, V, ex->ld(x.t[0]), st);
            if (rc) return rc;
            if (g_nccl.AllReduce(rowmax, rowmax, rows, 7, 2 /* max */, comm, st) != 0) return CAI_K_CUDA;
            rc = cai_ce_rowsum(P(0), rowmax, rowsum, rows, V, ex->ld(x.t[0]), st);
            if (rc) return rc;
            if (g_nccl.AllReduce(rowsum, rowsum, rows, 7, 0 /* sum */, comm, st) != 0) return CAI_K_CUDA;
            return cai_ce_grad_tp(P(0), (const int*)P(1), rowmax, rowsum, (float*)P(2), rows, V, ex->ld(x.t[0]), x.i[2],
                                  x.i[4], x.f[0], x.f[1], st);
        }
        case K_ADAMW: {
            const long long n = (static_cast<long long>(static_cast<uint32_t>(x.i[1])) << 32) | static_cast<uint32_t>(x.i[0]);
            const unsigned blocks = static_cast<unsigned>(((n + 3) / 4 + 255) / 256);
            adamw_dev_kernel<<<blocks, 256, 0, st>>>((float*)P(0), (float*)P(1), (float*)P(2), (const float*)P(3),
                                                     (__nv_bfloat16*)P(4), n, ex->hyper_dev, x.f[0]);
            return cudaGetLastError() == cudaSuccess ? 0 : CAI_K_CUDA;
        }
        case K_ZERO:
            return cudaMemsetAsync(P(0), 0, ex->tensors[x.t[0]].nbytes, st) == cudaSuccess ? 0 : CAI_K_CUDA;
        case K_ADD:
            return cai_add_bf16(P(0), P(1), P(2), x.i[0], st);
        case K_NCCL_ALL_REDUCE: case K_NCCL_REDUCE_SCATTER: case K_NCCL_ALL_GATHER: case K_NCCL_SEND: case K_NCCL_RECV: {
            const int group = x.i[3];
            if (group < 0 || group >= GROUP_COUNT || !ex->comms[group].comm) {
                set_last_error("op needs communicator %d which was not initialised", group);
                return CAI_K_BAD_ARG;
            }
            const Comm& c = ex->comms[group];
            const size_t count = (static_cast<size_t>(static_cast<uint32_t>(x.i[1])) << 32) | static_cast<uint32_t>(x.i[0]);
            const int dt = nccl_dtype(x.i[2]);
            int rc = 0;
            if (x.kernel == K_NCCL_ALL_REDUCE) rc = g_nccl.AllReduce(P(0), P(1), count, dt, 0, c.comm, st);
            else if (x.kernel == K_NCCL_REDUCE_SCATTER) rc = g_nccl.ReduceScatter(P(0), P(1), count, dt, 0, c.comm, st);
            else if (x.kernel == K_NCCL_ALL_GATHER) rc = g_nccl.AllGather(P(0), P(1), count, dt, c.comm, st);
            else {
                // pipeline hand-off: activations use the first communicator, gradients the second
                void* comm = (op.stream_id == ST_IO && c.comm2) ? c.comm2 : c.comm;
                if (x.kernel == K_NCCL_SEND) rc = g_nccl.Send(P(0), count, dt, x.i[4], comm, st);
                else rc = g_nccl.Recv(P(1), count, dt, x.i[4], comm, st);
            }
            if (rc != 0) {
                set_last_error("NCCL call failed: %s", g_nccl.GetErrorString(rc));
                return CAI_K_CUDA;
            }
            return 0;
        }
        case K_QUANT_FP8:
            if (x.flags & 1)
                return cai_quant_blocks_128x128(P(0), ex->ld(x.t[0]), P(1), ex->ld(x.t[1]), P(3), x.t[3] >= 0 ? ex->ld(x.t[3]) : 0,
                                                (float*)P(2), (float*)P(4), x.i[0], x.i[1], st);
            return cai_quant_rows_1x128(P(0), ex->ld(x.t[0]), P(1), ex->ld(x.t[1]), (float*)P(2), x.i[0], x.i[1], st);
        case K_GEMM_FP8:
            return cai_gemm_fp8_blockscaled(P(0), (const float*)P(4), P(1), (const float*)P(5), P(2), P(3), x.i[0], x.i[1], x.i[2],
                                            ex->ld(x.t[0]), ex->ld(x.t[1]), ex->ld(x.t[2]), x.t[3] >= 0 ? ex->ld(x.t[3]) : 0,
                                            x.flags >> 4, st);
        case K_FSDP_AG_GEMM: {
            if (!ex->has_peers[GROUP_DP] || ex->n_shard <= 0) {
                set_last_error("parameter gather needs the data-parallel peer table and a sharded plan");
                return CAI_K_BAD_ARG;
            }
            GatherJob job{};
            job.shard_off = ex->tensors[x.t[0]].offset;
            job.n_shard = ex->n_shard;
            job.lo = static_cast<long long>(static_cast<uint32_t>(x.i[0])) << 9;
            job.hi = static_cast<long long>(static_cast<uint32_t>(x.i[1])) << 9;
            job.dst = static_cast<__nv_bfloat16*>(P(1));
            job.reverse = (x.flags >> 1) & 1;
            job.group_kind = GROUP_DP;
            if (x.flags & 1) {
                job.n_copy = x.i[2] > 0 ? x.i[2] : (ex->ag_copy_ctas > 0 ? ex->ag_copy_ctas : 24);
                ex->pending_gather = job;
                ex->pending_seq = static_cast<uint32_t>(x.i[4]);
                ex->has_pending_gather = true;   // launched together with the next GEMM
                return 0;
            }
            job.n_copy = x.i[2] > 0 ? x.i[2] : 32;
            return cai_fsdp_gather(ex->peers[GROUP_DP], job, reinterpret_cast<const uint32_t*>(ex->hyper_dev) + 7,
                                   static_cast<uint32_t>(x.i[4]), st);
        }
        case K_MOE_ROUTE:
            if (x.flags & 1)
                return cai_moe_route_bwd((const float*)P(0), (const int*)P(1), (const float*)P(2), (const int*)P(3), P(4), x.i[0],
                                         x.i[1], x.i[2], st);
            return cai_moe_route_fwd((const float*)P(0), (int*)P(1), (float*)P(2), (int*)P(3), (int*)P(4), x.i[0], x.i[1], x.i[2],
                                     x.i[3], st);
        case K_MOE_DISPATCH_GEMM: case K_MOE_GEMM_COMBINE: {
            // The expert group has the members of the data-parallel group (ep == dp) or is this rank alone.
            PeerTable self{};
            const PeerTable* pt = nullptr;
            if (ex->has_peers[GROUP_EP]) pt = &ex->peers[GROUP_EP];
            else if (ex->hdr.ep > 1 && ex->has_peers[GROUP_DP] && ex->peers[GROUP_DP].size == static_cast<int>(ex->hdr.ep))
                pt = &ex->peers[GROUP_DP];
            else if (ex->hdr.ep <= 1) {
                int sig = -1;
                for (const NamedTensor& nt : ex->named)
                    if (!strcmp(nt.name, "@signals")) sig = nt.tensor;
                if (sig < 0) {
                    set_last_error("plan has no signal block");
                    return CAI_K_BAD_ARG;
                }
                self.base[0] = ex->arena;
                self.rank = 0;
                self.size = 1;
                self.sig_off = ex->tensors[sig].offset;
                pt = &self;
            } else {
                set_last_error("expert-parallel op needs the members' arenas (not exchanged)");
                return CAI_K_BAD_ARG;
            }
            const uint32_t* epoch_base = reinterpret_cast<const uint32_t*>(ex->hyper_dev) + 7;
            const uint32_t seq = static_cast<uint32_t>(x.i[4]);
            const int k = x.i[0], E = x.i[1], cap = x.i[2];
            if (x.kernel == K_MOE_DISPATCH_GEMM) {
                const int T = static_cast<int>(ex->shapes[static_cast<size_t>(x.t[0]) * 4]);
                const int H = static_cast<int>(ex->shapes[static_cast<size_t>(x.t[0]) * 4 + 1]);
                return cai_moe_dispatch(*pt, P(0), (const int*)P(1), (const int*)P(2), (const float*)P(3), (const int*)P(4),
                                        ex->tensors[x.t[5]].offset, ex->tensors[x.t[6]].offset, T, H, k, E, cap, epoch_base, seq,
                                        ex->counters_dev + 8, st);
            }
            const int T = static_cast<int>(ex->shapes[static_cast<size_t>(x.t[2]) * 4]);
            const int H = static_cast<int>(ex->shapes[static_cast<size_t>(x.t[5]) * 4 + 1]);
            return cai_moe_combine(*pt, P(0), P(1), (const int*)P(2), (const int*)P(3), (const float*)P(4),
                                   ex->tensors[x.t[5]].offset, P(6), (float*)P(7), T, H, k, E, cap, x.flags & 1, epoch_base, seq, st);
        }
        case K_AG_GEMM: case K_GEMM_RS: case K_RS_ADAMW: {
            const int group = x.i[3];
            if (group < 0 || group >= GROUP_COUNT || !ex->has_peers[group]) {
                set_last_error("fused op needs the peer table of communicator %d (arenas not exchanged)", group);
                return CAI_K_BAD_ARG;
            }
            const PeerTable& pt = ex->peers[group];
            const uint32_t* epoch_base = reinterpret_cast<const uint32_t*>(ex->hyper_dev) + 7;
            const uint32_t seq = static_cast<uint32_t>(x.i[4]);
            if (x.kernel == K_AG_GEMM) {
                const int T = x.i[0], N = x.i[1], K = x.i[2];
                return cai_fused_ag_gemm(pt, group, ex->tensors[x.t[0]].offset, ex->ld(x.t[0]), P(3), P(1), P(2), T, N, K,
                                         ex->ld(x.t[1]), ex->ld(x.t[2]), (x.flags >> 1) & 1, T / pt.size, epoch_base, seq,
                                         ex->ag_copy_ctas, st, (x.flags >> 4) & 0xF, P(5), x.t[5] >= 0 ? ex->ld(x.t[5]) : 0);
            }
            if (x.kernel == K_GEMM_RS) {
                const int T = x.i[0], N = x.i[1], K = x.i[2];
                return cai_fused_gemm_rs(pt, group, P(0), P(1), ex->tensors[x.t[4]].offset, P(2), P(3), T, N, K, ex->ld(x.t[0]),
                                         ex->ld(x.t[1]), ex->ld(x.t[2]), x.t[3] >= 0 ? ex->ld(x.t[3]) : 0, (x.flags >> 1) & 1,
                                         T / pt.size, epoch_base, seq, st);
            }
            const long long n_flat = (static_cast<long long>(static_cast<uint32_t>(x.i[1])) << 32) | static_cast<uint32_t>(x.i[0]);
            const long long n_shard = static_cast<uint32_t>(x.i[2]);
            if (x.flags & 2) {
                // a bucket [i0, i1) x 512 of the flat space: the record's tensors are the slices it touches (for the
                // hazard proof); the kernel indexes from the bases of the flat buffers
                const int fg = ex->flat_ids[0], fp = ex->flat_ids[1], fm = ex->flat_ids[2], f1 = ex->flat_ids[3], f2 = ex->flat_ids[4];
                if (fg < 0 || fp < 0 || fm < 0 || f1 < 0 || f2 < 0 || ex->n_rep <= 0) {
                    set_last_error("rs_adamw bucket: plan lacks the flat buffers");
                    return CAI_K_BAD_ARG;
                }
                const long long lo = static_cast<long long>(static_cast<uint32_t>(x.i[0])) << 9;
                const long long hi = static_cast<long long>(static_cast<uint32_t>(x.i[1])) << 9;
                const bool staged = (x.flags & 4) != 0;
                // sharded gradients: the members' staging buffer of the layer, and my slice of the accumulator moved
                // back to the start of the shard (the kernel indexes it like master)
                float* gacc = nullptr;
                if (staged && x.t[5] >= 0) {
                    const long long own_lo = lo > ex->peers[group].rank * ex->n_shard ? lo : ex->peers[group].rank * ex->n_shard;
                    gacc = static_cast<float*>(P(5)) - (own_lo - ex->peers[group].rank * ex->n_shard);
                }
                return cai_fused_rs_adamw(pt, staged ? ex->tensors[x.t[3]].offset : ex->tensors[fg].offset, ex->tensors[fp].offset,
                                          (float*)ex->ptr(fm), (float*)ex->ptr(f1), (float*)ex->ptr(f2), ex->n_rep, ex->n_shard,
                                          ex->hyper_dev, x.f[0], seq, ex->counters_dev, x.flags & 1, st, lo, hi, x.i[2], staged ? 1 : 0,
                                          gacc, (x.flags & 8) ? 1 : 0, (x.flags & 16) ? 1 : 0);
            }
            return cai_fused_rs_adamw(pt, ex->tensors[x.t[3]].offset, ex->tensors[x.t[4]].offset, (float*)P(0), (float*)P(1),
                                      (float*)P(2), n_flat, n_shard, ex->hyper_dev, x.f[0], seq, ex->counters_dev, x.flags & 1, st);
        }
        default:
            if (ex->fused_hook) return ex->fused_hook(ex->fused_ctx, ex, &x, static_cast<int>(op.stream_id), st);
            set_last_error("no launcher for kernel id %d", (int)x.kernel);
            return CAI_K_BAD_ARG;
    }
}

// Debug mode (cai_exec_set_debug / CAI_DEBUG_BOUNDS=1): before a record is launched, the extent every operand needs,
// worked out from the record's own dimensions (rows, columns, pitch, element size), is checked against the bytes
// the plan gives that tensor. A plan whose dimensions and tensor table disagree is refused with the op's index
// instead of letting a kernel run past a tensor into its neighbour in the arena.
struct Need { int t; long long rows, cols, ld, esize; };

bool operand_fits(const cai_exec* ex, const Need& n, const char** why) {
    if (n.t < 0 || n.rows <= 0 || n.cols <= 0) return true;
    const TensorDesc& td = ex->tensors[n.t];
    const long long ld = n.ld > 0 ? n.ld : n.cols;
    const unsigned long long need = (static_cast<unsigned long long>(n.rows - 1) * ld + n.cols) * n.esize;
    if (need > td.nbytes) {
        *why = "operand smaller than the extent the kernel addresses";
        return false;
    }
    if (td.offset + td.nbytes > ex->hdr.arena_bytes) {
        *why = "operand outside the arena";
        return false;
    }
    return true;
}

int check_operands(const cai_exec* ex, const ExecOp& x, size_t op_index) {
    std::vector<Need> needs;
    auto need = [&](int slot, long long rows, long long cols, long long esize, bool pitched = true) {
        Need n;
        n.t = x.t[slot];
        n.rows = rows; n.cols = cols; n.esize = esize;
        n.ld = (pitched && x.t[slot] >= 0) ? ex->ld(x.t[slot]) : 0;
        needs.push_back(n);
    };
    const long long i0 = x.i[0], i1 = x.i[1], i2 = x.i[2];
    switch (x.kernel) {
        case K_RMSNORM_FWD:
            need(0, i0, i1, 2); need(1, 1, i1, 2, false); need(2, i0, i1, 2); need(3, 1, i0, 4, false);
            break;
        case K_RMSNORM_BWD:
            need(0, i0, i1, 2); need(1, 1, i1, 2, false); need(2, 1, i0, 4, false); need(3, i0, i1, 2); need(4, i0, i1, 2);
            need(5, 1, i1, 4, false);
            break;
        case K_GEMM: {
            if ((x.flags & 0x100) || x.t[4] >= 0) break;   // grouped / ragged forms: not covered
            const int ta = x.flags & 1, tb = (x.flags >> 1) & 1, epi = (x.flags >> 4) & 0xF;
            const long long M = i0, N = i1, K = i2;
            if (ta) need(0, K, M, 2); else need(0, M, K, 2);
            if (tb) need(1, K, N, 2); else need(1, N, K, 2);
            if (epi == 4) { need(2, M, N, 2); need(3, M, N / 2, 2); }
            else if (epi == 5) { need(2, M, 2 * N, 2); need(3, M, 2 * N, 2); }
            else {
                need(2, M, N, (epi == 1 || epi == 2) ? 4 : 2);
                if (epi == 3) need(3, M, N, 2);
            }
            break;
        }
        case K_AG_GEMM: {
            const long long T = i0, N = i1, K = i2;
            const int tb = (x.flags >> 1) & 1, epi = (x.flags >> 4) & 0xF;
            need(3, T, K, 2);
            if (tb) need(1, K, N, 2); else need(1, N, K, 2);
            need(2, T, epi == 5 ? 2 * N : N, 2);
            if (epi == 4) need(5, T, N / 2, 2);
            if (epi == 5) need(5, T, 2 * N, 2);
            break;
        }
        case K_GEMM_RS: {
            const long long T = i0, N = i1, K = i2;
            const int tb = (x.flags >> 1) & 1;
            need(0, T, K, 2);
            if (tb) need(1, K, N, 2); else need(1, N, K, 2);
            need(4, T, N, 2);
            break;
        }
        case K_ROPE: need(0, i0, (static_cast<long long>(x.i[2]) + x.i[3]) * x.i[4], 2); break;
        case K_ATTN_FWD: case K_ATTN_BWD: {
            const long long rows = i0 * i1, nh = i2, nkv = x.i[3], hd = x.i[4];
            need(0, rows, (nh + 2 * nkv) * hd, 2);
            need(1, rows, nh * hd, 2);
            if (x.kernel == K_ATTN_FWD) need(2, nh * i0, i1, 4, false);
            else { need(2, rows, nh * hd, 2); need(5, rows, (nh + 2 * nkv) * hd, 2); }
            break;
        }
        case K_SWIGLU_FWD: need(0, i0, 2 * i1, 2); need(1, i0, i1, 2); break;
        case K_SWIGLU_BWD: need(0, i0, 2 * i1, 2); need(1, i0, i1, 2); need(2, i0, 2 * i1, 2); break;
        case K_CROSS_ENTROPY: case K_CROSS_ENTROPY_TP: need(0, i0, i1, 2); need(1, 1, i0, 4, false); break;
        case K_EMBED_FWD: need(0, 1, i0, 4, false); need(2, i0, i1, 2); break;
        case K_EMBED_BWD: need(0, 1, i0, 4, false); need(1, i0, i1, 2); break;
        default: break;
    }
    for (const Need& n : needs) {
        const char* why = nullptr;
        if (!operand_fits(ex, n, &why)) {
            set_last_error("debug bounds: op %zu (kernel %d): tensor %d (%llu bytes) %s (%lld x %lld, pitch %lld, %lld-byte elements)",
                           op_index, (int)x.kernel, n.t, (unsigned long long)ex->tensors[n.t].nbytes, why, n.rows, n.cols,
                           n.ld > 0 ? n.ld : n.cols, n.esize);
            return CAI_K_BAD_ARG;
        }
    }
    return 0;
}

// How many kernels of this library one exec record launches (memsets and NCCL calls are not ours).
int own_kernels_of(const ExecOp& x) {
    const uint16_t k = x.kernel;
    if (k == K_ZERO || (k >= K_NCCL_ALL_REDUCE && k <= K_NCCL_RECV)) return 0;
    if (k == K_FSDP_AG_GEMM && (x.flags & 1)) return 0;            // rides in the GEMM that follows
    if (k == K_ATTN_BWD) return x.flags ? __builtin_popcount(x.flags) : 3;
    if (k == K_CROSS_ENTROPY_TP) return 3;
    if (k == K_RMSNORM_BWD) return x.i[1] <= 8192 ? 2 : 3;         // one sweep + reduce, or dg / reduce / dx
    if (k == K_MOE_ROUTE && !(x.flags & 1)) return 2;              // top-k, then slots in token order
    return 1;
}

// names of the kernel ids, for NVTX ranges (same order as the enum in plan/formats.h)
const char* kernel_label(uint16_t k) {
    static const char* n[K_COUNT] = {"none", "embed_fwd", "embed_bwd", "rmsnorm_fwd", "rmsnorm_bwd", "gemm", "rope", "attn_fwd",
                                     "attn_bwd", "swiglu_fwd", "swiglu_bwd", "cross_entropy", "adamw", "zero", "nccl_all_reduce",
                                     "nccl_reduce_scatter", "nccl_all_gather", "nccl_all_to_all", "nccl_send", "nccl_recv",
                                     "gemm_rs", "ag_gemm", "rs_adamw", "fsdp_ag_gemm", "moe_route", "moe_dispatch", "moe_combine",
                                     "load_tokens", "add", "cross_entropy_tp", "quant_fp8", "gemm_fp8"};
    return k < K_COUNT ? n[k] : "?";
}

int replay(cai_exec* ex) {
    cudaStream_t hi = ex->streams[ST_COMPUTE_HI];
    // fork: every stream starts after everything already queued on compute_hi
    cudaEventRecord(ex->fork_ev, hi);
    for (int s = 1; s < ST_COUNT; ++s) cudaStreamWaitEvent(ex->streams[s], ex->fork_ev, 0);
    ex->launches = 0;
    for (size_t i = 0; i < ex->ops.size(); ++i) {
        const Op& op = ex->ops[i];
        cudaStream_t st = ex->streams[op.stream_id];
        if (op.kind == OP_EVENT_RECORD) {
            if (cudaEventRecord(ex->events[op.aux0], st) != cudaSuccess) return CAI_K_CUDA;
            continue;
        }
        if (op.kind == OP_EVENT_WAIT) {
            if (cudaStreamWaitEvent(st, ex->events[op.aux0], 0) != cudaSuccess) return CAI_K_CUDA;
            continue;
        }
        if (!op.exec) continue;
        TraceRec* tr = nullptr;
        if (ex->trace_on && !ex->use_graph) {
            TraceRec r;
            r.op = static_cast<uint32_t>(i);
            cudaEventCreate(&r.start);
            cudaEventCreate(&r.stop);
            ex->trace.push_back(r);
            tr = &ex->trace.back();
            cudaEventRecord(tr->start, st);
        }
        if (ex->debug_bounds) {
            const int brc = check_operands(ex, ex->exec[op.exec - 1], i);
            if (brc != 0) return brc;
        }
        if (ex->nvtx_on) nvtxRangePushA(kernel_label(ex->exec[op.exec - 1].kernel));
        const int rc = run_op(ex, op, ex->exec[op.exec - 1], st);
        if (ex->nvtx_on) nvtxRangePop();
        if (rc != 0) return rc;
        {
            ex->launches += own_kernels_of(ex->exec[op.exec - 1]);
        }
        if (tr) cudaEventRecord(tr->stop, st);
    }
    // join: compute_hi waits for every other stream
    for (int s = 1; s < ST_COUNT; ++s) {
        cudaEventRecord(ex->join_ev[s], ex->streams[s]);
        cudaStreamWaitEvent(hi, ex->join_ev[s], 0);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : CAI_K_CUDA;
}

}  // namespace

CAI_API int cai_exec_create(cai_exec** out, const void* plan_bytes, size_t nbytes, void* arena_base,
                            void* const* caller_streams) {
    auto ex = new cai_exec();
    const uint8_t* p = static_cast<const uint8_t*>(plan_bytes);
    const uint8_t* end = p + nbytes;
    auto take = [&](void* dst, size_t n) {
        if (p + n > end) return false;
        memcpy(dst, p, n);
        p += n;
        return true;
    };
    bool ok = take(&ex->hdr, sizeof ex->hdr) && ex->hdr.magic == kPlanMagic && ex->hdr.version == 2;
    if (ok) {
        ex->tensors.resize(ex->hdr.num_tensors);
        ex->groups.resize(ex->hdr.num_groups);
        ex->ops.resize(ex->hdr.num_ops);
        ok = take(ex->tensors.data(), ex->tensors.size() * sizeof(TensorDesc)) &&
             take(ex->groups.data(), ex->groups.size() * sizeof(CommGroup)) &&
             take(ex->ops.data(), ex->ops.size() * sizeof(Op)) && take(&ex->xhdr, sizeof ex->xhdr) &&
             ex->xhdr.magic == kExecMagic && take(&ex->train, sizeof ex->train) && take(&ex->model, sizeof ex->model);
    }
    if (ok) {
        ex->exec.resize(ex->xhdr.num_exec);
        ex->named.resize(ex->xhdr.num_named);
        ex->shapes.resize(static_cast<size_t>(ex->hdr.num_tensors) * 4);
        ok = take(ex->exec.data(), ex->exec.size() * sizeof(ExecOp)) &&
             take(ex->named.data(), ex->named.size() * sizeof(NamedTensor)) &&
             take(ex->shapes.data(), ex->shapes.size() * sizeof(uint32_t));
    }
    if (!ok) {
        set_last_error("not a version-2 plan (or truncated)");
        delete ex;
        return CAI_K_BAD_ARG;
    }
    for (const TensorDesc& t : ex->tensors)
        if (t.offset + t.nbytes > ex->hdr.arena_bytes) {
            set_last_error("tensor outside the arena");
            delete ex;
            return CAI_K_BAD_ARG;
        }
    for (const Op& o : ex->ops)
        if (o.stream_id >= ST_COUNT || ((o.kind == OP_EVENT_RECORD || o.kind == OP_EVENT_WAIT) && o.aux0 >= ex->hdr.num_events) ||
            o.exec > ex->exec.size()) {
            set_last_error("malformed op table");
            delete ex;
            return CAI_K_BAD_ARG;
        }
    ex->arena = static_cast<uint8_t*>(arena_base);
    ex->device = current_device();
    if (const char* dbg = getenv("CAI_DEBUG_BOUNDS")) ex->debug_bounds = *dbg && *dbg != '0';
    if (ex->train.wait_limit_ms) cai_set_wait_limit_us(ex->train.wait_limit_ms * 1000u);
    int lo_prio = 0, hi_prio = 0;
    cudaDeviceGetStreamPriorityRange(&lo_prio, &hi_prio);
    for (int s = 0; s < ST_COUNT; ++s) {
        const int prio = (s == ST_COMPUTE_HI || s == ST_COMM_TP) ? hi_prio : lo_prio;
        if (caller_streams && caller_streams[s]) {
            // streams owned by the caller (e.g. a framework's stream pool) are used, never destroyed
            ex->streams[s] = static_cast<cudaStream_t>(caller_streams[s]);
        } else if (cudaStreamCreateWithPriority(&ex->streams[s], cudaStreamNonBlocking, prio) == cudaSuccess) {
            ex->owns_stream[s] = true;
        } else {
            set_last_error("stream creation failed");
            delete ex;
            return CAI_K_CUDA;
        }
        cudaEventCreateWithFlags(&ex->join_ev[s], cudaEventDisableTiming);
    }
    cudaEventCreateWithFlags(&ex->fork_ev, cudaEventDisableTiming);
    ex->events.resize(ex->hdr.num_events);
    for (cudaEvent_t& e : ex->events) cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
    bool dev_ok = true;
    for (int s = 0; s < ST_COUNT; ++s) dev_ok = dev_ok && ex->join_ev[s] != nullptr;
    dev_ok = dev_ok && ex->fork_ev != nullptr;
    for (cudaEvent_t e : ex->events) dev_ok = dev_ok && e != nullptr;
    dev_ok = dev_ok && cudaMalloc(&ex->hyper_dev, 8 * sizeof(float)) == cudaSuccess;
    dev_ok = dev_ok && cudaMalloc(&ex->counters_dev, 256 * sizeof(unsigned int)) == cudaSuccess;
    dev_ok = dev_ok && cudaMemset(ex->counters_dev, 0, 256 * sizeof(unsigned int)) == cudaSuccess;
    dev_ok = dev_ok && cudaMemset(ex->hyper_dev, 0, 8 * sizeof(float)) == cudaSuccess;
    dev_ok = dev_ok && cudaMallocHost(&ex->hyper_host, cai_exec::kHyperSlots * 8 * sizeof(float)) == cudaSuccess;
    for (int i = 0; i < cai_exec::kHyperSlots && dev_ok; ++i)
        dev_ok = cudaEventCreateWithFlags(&ex->hyper_ev[i], cudaEventDisableTiming) == cudaSuccess;
    if (!dev_ok) {
        set_last_error("executor set-up failed (event / device / pinned allocation): %s", cudaGetErrorString(cudaGetLastError()));
        cai_exec_destroy(ex);
        return CAI_K_CUDA;
    }
    {
        uint32_t fused = 0;
        for (const ExecOp& x : ex->exec)
            if (x.kernel == K_AG_GEMM || x.kernel == K_GEMM_RS || x.kernel == K_RS_ADAMW || x.kernel == K_MOE_DISPATCH_GEMM ||
                x.kernel == K_MOE_GEMM_COMBINE || x.kernel == K_FSDP_AG_GEMM)
                ++fused;
        static const char* const flat_names[5] = {"@flat_grad", "@flat_param", "@flat_master", "@flat_m", "@flat_v"};
        for (const NamedTensor& nt : ex->named) {
            if (!strcmp(nt.name, "@flat_split")) {
                ex->n_shard = static_cast<long long>(nt.rows) << 9;
                ex->n_rep = static_cast<long long>(nt.master) << 9;
            }
            for (int k = 0; k < 5; ++k)
                if (!strcmp(nt.name, flat_names[k])) ex->flat_ids[k] = nt.tensor;
        }
        ex->epochs_per_step = 2 * fused + 2;
    }
    *out = ex;
    return 0;
}

CAI_API void cai_exec_destroy(cai_exec* ex) {
    if (!ex) return;
    cudaDeviceSynchronize();
    if (ex->graph) cudaGraphExecDestroy(ex->graph);
    for (TraceRec& r : ex->trace) { cudaEventDestroy(r.start); cudaEventDestroy(r.stop); }
    for (cudaEvent_t e : ex->events) cudaEventDestroy(e);
    for (int s = 0; s < ST_COUNT; ++s) {
        if (ex->join_ev[s]) cudaEventDestroy(ex->join_ev[s]);
        if (ex->streams[s] && ex->owns_stream[s]) cudaStreamDestroy(ex->streams[s]);
    }
    if (ex->fork_ev) cudaEventDestroy(ex->fork_ev);
    for (Comm& c : ex->comms) {
        if (c.comm && g_nccl.CommDestroy) g_nccl.CommDestroy(c.comm);
        if (c.comm2 && g_nccl.CommDestroy) g_nccl.CommDestroy(c.comm2);
    }
    for (cudaEvent_t e : ex->hyper_ev)
        if (e) cudaEventDestroy(e);
    if (ex->hyper_dev) cudaFree(ex->hyper_dev);
    if (ex->counters_dev) cudaFree(ex->counters_dev);
    if (ex->hyper_host) cudaFreeHost(ex->hyper_host);
    delete ex;
}

CAI_API int cai_nccl_unique_id(const char* libpath, void* id128) {
    if (!nccl_load(libpath)) return CAI_K_CUDA;
    const int rc = g_nccl.GetUniqueId(id128);
    if (rc != 0) {
        set_last_error("ncclGetUniqueId: %s", g_nccl.GetErrorString(rc));
        return CAI_K_CUDA;
    }
    return 0;
}

CAI_API int cai_exec_init_comm(cai_exec* ex, const char* libpath, int group_kind, const void* id128, const void* id128_second,
                               int nranks, int rank) {
    if (group_kind < 0 || group_kind >= GROUP_COUNT) return CAI_K_BAD_ARG;
    if (!nccl_load(libpath)) return CAI_K_CUDA;
    Comm& c = ex->comms[group_kind];
    c.rank = rank;
    c.size = nranks;
    NcclId id;
    memcpy(&id, id128, sizeof id);
    int rc = g_nccl.CommInitRank(&c.comm, nranks, id, rank);
    if (rc == 0 && id128_second) {
        memcpy(&id, id128_second, sizeof id);
        rc = g_nccl.CommInitRank(&c.comm2, nranks, id, rank);
    }
    if (rc != 0) {
        set_last_error("ncclCommInitRank: %s", g_nccl.GetErrorString(rc));
        return CAI_K_CUDA;
    }
    return 0;
}

// Arena bases of the members of a communicator as mapped in this process (bases[rank] is the local
// arena). Enables the fused compute+collective kernels of that communicator.
CAI_API int cai_exec_set_peers(cai_exec* ex, int group_kind, int n, void* const* bases, int rank) {
    if (group_kind < 0 || group_kind >= GROUP_COUNT || n < 1 || n > kMaxPeers || rank < 0 || rank >= n) return CAI_K_BAD_ARG;
    int sig = -1;
    for (const NamedTensor& nt : ex->named)
        if (!strcmp(nt.name, "@signals")) sig = nt.tensor;
    if (sig < 0 || ex->tensors[sig].nbytes < kSigBytes) {
        set_last_error("plan has no signal block");
        return CAI_K_BAD_ARG;
    }
    PeerTable& pt = ex->peers[group_kind];
    for (int i = 0; i < n; ++i) pt.base[i] = static_cast<uint8_t*>(bases[i]);
    pt.rank = rank;
    pt.size = n;
    pt.sig_off = ex->tensors[sig].offset;
    ex->has_peers[group_kind] = true;
    return 0;
}
CAI_API void cai_exec_set_ag_copy_ctas(cai_exec* ex, int n) { ex->ag_copy_ctas = n; }

CAI_API void* cai_exec_stream(cai_exec* ex, int stream_id) {
    return stream_id >= 0 && stream_id < ST_COUNT ? ex->streams[stream_id] : nullptr;
}
CAI_API void* cai_exec_tensor_ptr(cai_exec* ex, int tensor) {
    return tensor >= 0 && static_cast<size_t>(tensor) < ex->tensors.size() ? ex->ptr(tensor) : nullptr;
}
CAI_API long long cai_exec_tensor_ld(cai_exec* ex, int tensor) { return ex->ld(tensor); }
CAI_API unsigned long long cai_exec_tensor_bytes(cai_exec* ex, int tensor) { return ex->tensors[tensor].nbytes; }
CAI_API int cai_exec_group_rank(cai_exec* ex, int kind) { return ex->comms[kind].rank; }
CAI_API int cai_exec_group_size(cai_exec* ex, int kind) { return ex->comms[kind].size; }
CAI_API unsigned long long cai_exec_launches(cai_exec* ex) { return ex->launches; }
CAI_API void cai_exec_set_fused_hook(cai_exec* ex, cai_fused_hook_t hook, void* ctx) {
    ex->fused_hook = hook;
    ex->fused_ctx = ctx;
}
CAI_API void cai_exec_set_sm_limit(cai_exec* ex, int sms) { ex->sm_limit_hi = sms; }
CAI_API float* cai_exec_hyper(cai_exec* ex) { return ex->hyper_dev; }

// Enqueue one optimizer step (all microbatches, forward + backward + update). `step` is the
// 1-based AdamW step count. Returns after enqueueing; the caller synchronises when it wants
// the loss.
CAI_API int cai_exec_step(cai_exec* ex, int step, float lr) {
    cudaStream_t hi = ex->streams[ST_COMPUTE_HI];
    const unsigned slot = ex->hyper_next++ % cai_exec::kHyperSlots;
    if (ex->hyper_used[slot] && cudaEventSynchronize(ex->hyper_ev[slot]) != cudaSuccess) return CAI_K_CUDA;
    float* h = ex->hyper_host + slot * 8;
    const TrainSpec& t = ex->train;
    h[0] = lr; h[1] = t.beta1; h[2] = t.beta2; h[3] = t.adam_eps; h[4] = t.weight_decay;
    h[5] = 1.f - powf(t.beta1, static_cast<float>(step));
    h[6] = 1.f - powf(t.beta2, static_cast<float>(step));
    // epoch base of this step's fused kernels: grows by a fixed stride per step, never resets
    reinterpret_cast<uint32_t*>(h)[7] = static_cast<uint32_t>(step) * ex->epochs_per_step;
    if (cudaMemcpyAsync(ex->hyper_dev, h, 8 * sizeof(float), cudaMemcpyHostToDevice, hi) != cudaSuccess) return CAI_K_CUDA;
    if (cudaEventRecord(ex->hyper_ev[slot], hi) != cudaSuccess) return CAI_K_CUDA;
    ex->hyper_used[slot] = true;
    if (ex->use_graph) {
        if (!ex->graph) {
            cudaGraph_t g = nullptr;
            if (cudaStreamBeginCapture(hi, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
                set_last_error("cudaStreamBeginCapture failed");
                return CAI_K_CUDA;
            }
            const int rc = replay(ex);
            const cudaError_t ce = cudaStreamEndCapture(hi, &g);
            if (rc != 0 || ce != cudaSuccess || !g) {
                if (rc == 0) set_last_error("graph capture failed: %s", cudaGetErrorString(ce));
                if (g) cudaGraphDestroy(g);
                return rc ? rc : CAI_K_CUDA;
            }
            const cudaError_t ie = cudaGraphInstantiate(&ex->graph, g, 0);
            cudaGraphDestroy(g);
            if (ie != cudaSuccess) {
                set_last_error("cudaGraphInstantiate failed: %s", cudaGetErrorString(ie));
                return CAI_K_CUDA;
            }
        }
        return cudaGraphLaunch(ex->graph, hi) == cudaSuccess ? 0 : CAI_K_CUDA;
    }
    if (ex->trace_on) {
        for (TraceRec& r : ex->trace) { cudaEventDestroy(r.start); cudaEventDestroy(r.stop); }
        ex->trace.clear();
        ex->trace.reserve(ex->ops.size());
    }
    return replay(ex);
}

CAI_API int cai_exec_sync(cai_exec* ex) {
    return cudaStreamSynchronize(ex->streams[ST_COMPUTE_HI]) == cudaSuccess ? 0 : CAI_K_CUDA;
}

CAI_API int cai_exec_use_graph(cai_exec* ex, int on) {
    ex->use_graph = on != 0;
    if (!on && ex->graph) {
        cudaGraphExecDestroy(ex->graph);
        ex->graph = nullptr;
    }
    return 0;
}

CAI_API int cai_exec_trace_enable(cai_exec* ex, int on) {
    ex->trace_on = on != 0;
    return 0;
}
CAI_API int cai_exec_set_debug(cai_exec* ex, int on) {
    ex->debug_bounds = on != 0;
    return 0;
}
CAI_API int cai_exec_nvtx_enable(cai_exec* ex, int on) {
    ex->nvtx_on = on != 0;
    return 0;
}

// Measured timeline of the last traced step: one record per op with start / end in seconds
// relative to the first op. Returns the number of records written.
CAI_API int cai_exec_trace_read(cai_exec* ex, cai_exec_trace_rec* out, int cap) {
    if (ex->trace.empty()) return 0;
    cudaDeviceSynchronize();
    int n = 0;
    for (const TraceRec& r : ex->trace) {
        if (n >= cap) break;
        float a = 0.f, b = 0.f;
        cudaEventElapsedTime(&a, ex->trace[0].start, r.start);
        cudaEventElapsedTime(&b, ex->trace[0].start, r.stop);
        const Op& op = ex->ops[r.op];
        out[n].op_index = r.op;
        out[n].kind = op.kind;
        out[n].stream = op.stream_id;
        out[n].start_s = a * 1e-3;
        out[n].end_s = b * 1e-3;
        out[n].bytes = op.bytes;
        out[n].flops = op.flops;
        ++n;
    }
    return n;
}
