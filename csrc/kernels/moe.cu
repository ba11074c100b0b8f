// moe.cu - mixture-of-experts routing and the expert-parallel token exchange.
//
// Router: softmax over the experts, top-k selection, weights renormalised over the chosen k.
// Exchange: experts are sharded over the expert-parallel group; every member keeps, per local
// expert and per source member, a slab of `cap` rows inside its arena. Dispatch is ONE kernel that
// permutes token rows by expert and writes them straight into the owning member's slab with peer
// stores over NVLink (optionally scaled per row, which is what the backward of the combine needs),
// publishes the row counts, zero-pads the ragged tail the weight-gradient GEMM will read, and
// performs the group handshake. Combine is ONE kernel that pulls each token's k expert outputs from
// the owners' slabs with peer loads and accumulates them weighted into the residual stream. The
// expert GEMMs in between run over the slabs with the segmented form of the tcgen05 GEMM.
// No NCCL all-to-all is involved. With a group of one member the same kernels do the local permute.
//
// The reference only prices two ALL_TO_ALL ops per layer in its cost model (src/model.c:463-475)
// and has no routing, dispatch or combine code at all.
#include <math.h>

#include "../comm/moe.h"
#include "../comm/peer.cuh"
#include "../plan/formats.h"
#include "cai_kernels.h"
#include "host_common.h"
#include "norm_kernels.cuh"
#include "sm100.cuh"

namespace cai {

constexpr int kMoeMaxK = 8;
constexpr int kMoeMaxEPerLane = 8;  // experts <= 256

// ------------------------------------------------------------------ router forward
// One warp per token. logits f32 [T, E].
__global__ void __launch_bounds__(256)
moe_route_fwd_kernel(const float* __restrict__ logits, int* __restrict__ idx, float* __restrict__ w, int* __restrict__ pos,
                     int* __restrict__ counts, int T, int E, int k, int cap) {
    const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    const int per = E >> 5;
    float p[kMoeMaxEPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMoeMaxEPerLane; ++i)
        if (i < per) {
            p[i] = logits[static_cast<long long>(t) * E + i * 32 + lane];
            mx = fmaxf(mx, p[i]);
        }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMoeMaxEPerLane; ++i)
        if (i < per) {
            p[i] = __expf(p[i] - mx);
            sum += p[i];
        }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    unsigned taken = 0;  // bit i: my i-th expert has been selected
    float sel_p = 0.f;   // lane s keeps the probability of the s-th choice
    int sel_e = 0;
    float S = 0.f;
    for (int s = 0; s < k; ++s) {
        float best = -1.f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMoeMaxEPerLane; ++i)
            if (i < per && !(taken >> i & 1) && p[i] > best) {
                best = p[i];
                best_e = i * 32 + lane;
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) {
                best = ob;
                best_e = oe;
            }
        }
        if ((best_e & 31) == lane) taken |= 1u << (best_e >> 5);
        if (lane == s) {
            sel_p = best * inv;
            sel_e = best_e;
        }
        S += best * inv;
    }
    if (lane < k) {
        idx[t * k + lane] = sel_e;
        w[t * k + lane] = sel_p / S;
    }
}

// Slot of every (token, choice) inside its expert's slab, in token order: pos[i] = how many earlier entries
// of idx chose the same expert, or -1 past the slab's capacity (the token skips that expert). One CTA per
// expert scans idx front to back, so which tokens are dropped and the row order inside a slab are the same in
// every run (an atomic counter per expert would hand out slots in arrival order). counts[e] is the number
// of entries that chose e, dropped ones included.
__global__ void __launch_bounds__(256)
moe_assign_slots_kernel(const int* __restrict__ idx, int* __restrict__ pos, int* __restrict__ counts, int n, int cap) {
    __shared__ int warp_tot[8];
    const int e = blockIdx.x, lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
    int base = 0;
    for (int i0 = 0; i0 < n; i0 += 256 * 8) {
        const int i = i0 + threadIdx.x * 8;
        unsigned mask = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (i + j < n && idx[i + j] == e) mask |= 1u << j;
        const int mine = __popc(mask);
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) warp_tot[wp] = incl;
        __syncthreads();
        int before = 0, total = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            if (q < wp) before += warp_tot[q];
            total += warp_tot[q];
        }
        int slot = base + before + incl - mine;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (mask >> j & 1) {
                pos[i + j] = slot < cap ? slot : -1;
                ++slot;
            }
        base += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = base;
}

// ------------------------------------------------------------------ router backward
// dlogits (bf16 [T, E]) from dw (f32 [T, k]); softmax probabilities are recomputed from the logits.
__global__ void __launch_bounds__(256)
moe_route_bwd_kernel(const float* __restrict__ logits, const int* __restrict__ idx, const float* __restrict__ dw,
                     const int* __restrict__ pos, __nv_bfloat16* __restrict__ dlogits, int T, int E, int k) {
    const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    const int per = E >> 5;
    float p[kMoeMaxEPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMoeMaxEPerLane; ++i)
        if (i < per) {
            p[i] = logits[static_cast<long long>(t) * E + i * 32 + lane];
            mx = fmaxf(mx, p[i]);
        }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMoeMaxEPerLane; ++i)
        if (i < per) {
            p[i] = __expf(p[i] - mx);
            sum += p[i];
        }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < kMoeMaxEPerLane; ++i)
        if (i < per) p[i] /= sum;
    // lane s < k owns choice s
    int e = 0;
    float pe = 0.f, g = 0.f;
    if (lane < k) {
        e = idx[t * k + lane];
        g = pos[t * k + lane] >= 0 ? dw[t * k + lane] : 0.f;  // dropped choices carry no gradient
    }
    // probability of each choice, fetched from the lane that holds that expert
    for (int s = 0; s < k; ++s) {
        const int es = __shfl_sync(0xffffffffu, e, s);
        float v = 0.f;
#pragma unroll
        for (int i = 0; i < kMoeMaxEPerLane; ++i)
            if (i < per && i * 32 + lane == es) v = p[i];
        v = warp_sum(v);
        if (lane == s) pe = v;
    }
    const float S = warp_sum(lane < k ? pe : 0.f);
    const float wv = pe / S;                                  // w_s
    const float gw = warp_sum(lane < k ? g * wv : 0.f);       // sum_j dw_j w_j
    const float dp = lane < k ? (g - gw) / S : 0.f;           // d loss / d p_s for the chosen experts
    const float gp = warp_sum(lane < k ? dp * pe : 0.f);      // sum_i dp_i p_i
    float dl[kMoeMaxEPerLane];
#pragma unroll
    for (int i = 0; i < kMoeMaxEPerLane; ++i)
        if (i < per) dl[i] = -p[i] * gp;
    for (int s = 0; s < k; ++s) {
        const int es = __shfl_sync(0xffffffffu, e, s);
        const float dps = __shfl_sync(0xffffffffu, dp, s);
#pragma unroll
        for (int i = 0; i < kMoeMaxEPerLane; ++i)
            if (i < per && i * 32 + lane == es) dl[i] += p[i] * dps;
    }
#pragma unroll
    for (int i = 0; i < kMoeMaxEPerLane; ++i)
        if (i < per) dlogits[static_cast<long long>(t) * E + i * 32 + lane] = __float2bfloat16(dl[i]);
}

// ------------------------------------------------------------------ dispatch
struct MoeDispatchParams {
    const __nv_bfloat16* rows;   // [T, H] local source rows
    const int* idx;              // [T, k]
    const int* pos;              // [T, k]
    const float* scale;          // [T, k] or null
    const int* counts;           // [E] tokens this member routed to each expert (may exceed cap)
    unsigned long long slab_off; // arena offset of the destination slab [E_l * ep * cap, H] on every member
    unsigned long long cnt_off;  // arena offset of the int32 [E_l * ep] count table on every member
    int T, H, k, E, E_l, cap;
    const uint32_t* epoch_base;
    uint32_t seq;
    unsigned int* done_counter;
    int* status;
};

__global__ void __launch_bounds__(256) moe_dispatch_kernel(const PeerTable pt, const MoeDispatchParams p) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const long long gw = static_cast<long long>(blockIdx.x) * warps_per_cta + (threadIdx.x >> 5);
    const long long nwarps = static_cast<long long>(gridDim.x) * warps_per_cta;
    const int hv = p.H >> 3;
    // (1) counts and zero padding of the ragged tails: warp e handles expert e
    for (long long e = gw; e < p.E; e += nwarps) {
        const int dst = static_cast<int>(e) / p.E_l, el = static_cast<int>(e) % p.E_l;
        const int cnt = p.counts[e] < p.cap ? p.counts[e] : p.cap;
        const int sub = el * pt.size + pt.rank;
        if (lane == 0) reinterpret_cast<int*>(pt.base[dst] + p.cnt_off)[sub] = cnt;
        const int pad_end = ((cnt + 127) & ~127) < p.cap ? ((cnt + 127) & ~127) : p.cap;
        __nv_bfloat16* slab = reinterpret_cast<__nv_bfloat16*>(pt.base[dst] + p.slab_off) + static_cast<long long>(sub) * p.cap * p.H;
        for (int r = cnt; r < pad_end; ++r)
            for (int c = lane; c < hv; c += 32) reinterpret_cast<uint4*>(slab + static_cast<long long>(r) * p.H)[c] = make_uint4(0, 0, 0, 0);
    }
    // (2) one warp per (token, choice): copy the row into the owner's slab
    const long long pairs = static_cast<long long>(p.T) * p.k;
    for (long long i = gw; i < pairs; i += nwarps) {
        const int ps = p.pos[i];
        if (ps < 0) continue;
        const int e = p.idx[i];
        const int dst = e / p.E_l, el = e % p.E_l;
        const long long t = i / p.k;
        const uint4* src = reinterpret_cast<const uint4*>(p.rows + t * p.H);
        uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(pt.base[dst] + p.slab_off) +
                                              (static_cast<long long>(el * pt.size + pt.rank) * p.cap + ps) * p.H);
        const float sc = p.scale ? p.scale[i] : 1.f;
        // four independent 16-byte loads in flight per lane before the first store
        for (int c0 = lane; c0 < hv; c0 += 128) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (c0 + 32 * u < hv) v[u] = src[c0 + 32 * u];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (c0 + 32 * u >= hv) break;
                if (p.scale) {
                    float f[8];
                    unpack8(v[u], f);
#pragma unroll
                    for (int q = 0; q < 8; ++q) f[q] *= sc;
                    v[u] = pack8(f);
                }
                out[c0 + 32 * u] = v[u];
            }
        }
    }
    // (3) handshake by the last CTA: everything this member sends has been issued and fenced; when
    // the kernel retires, everything the other members send to this one has landed as well
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int ticket = atomicAdd(p.done_counter, 1u);
        if (ticket == gridDim.x - 1) {
            *p.done_counter = 0;
            __threadfence();
            const uint32_t epoch = *p.epoch_base + 2 * p.seq;
            signal_all(pt, GROUP_EP, kSigEntry + pt.rank, epoch);
            wait_all(pt, GROUP_EP, kSigEntry, epoch, p.status);
        }
    }
}

// ------------------------------------------------------------------ combine (gather)
struct MoeCombineParams {
    const __nv_bfloat16* base;   // [T, H] residual added to the result, or null
    __nv_bfloat16* out;          // [T, H]
    const int* idx;
    const int* pos;
    const float* w;              // [T, k] weights, or null for plain sums
    unsigned long long slab_off; // arena offset of the expert output slab on every member
    const __nv_bfloat16* dot_with;  // dw mode: [T, H] rows to take dot products with
    float* dw;                      // dw mode: [T, k] output
    int T, H, k, E_l, cap;
    int announce;                // 1: publish "my slab is ready" and wait for every member first
    const uint32_t* epoch_base;
    uint32_t seq;
    int* status;
};

__global__ void __launch_bounds__(256) moe_combine_kernel(const PeerTable pt, const MoeCombineParams p) {
    __shared__ int ok_s;
    if (p.announce) {
        const uint32_t epoch = *p.epoch_base + 2 * p.seq;
        if (threadIdx.x == 0) {
            if (blockIdx.x == 0) signal_all(pt, GROUP_EP, kSigExit + pt.rank, epoch);
            ok_s = wait_all(pt, GROUP_EP, kSigExit, epoch, p.status) ? 1 : 0;
        }
        __syncthreads();
        if (!ok_s) return;
    }
    const int lane = threadIdx.x & 31;
    const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (t >= p.T) return;
    const int hv = p.H >> 3;
    const uint4* rows[kMoeMaxK];
    float ws[kMoeMaxK];
#pragma unroll
    for (int s = 0; s < kMoeMaxK; ++s) {
        rows[s] = nullptr;
        ws[s] = 0.f;
        if (s < p.k) {
            const int ps = p.pos[t * p.k + s];
            if (ps >= 0) {
                const int e = p.idx[t * p.k + s];
                const int owner = e / p.E_l, el = e % p.E_l;
                rows[s] = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(pt.base[owner] + p.slab_off) +
                                                         (static_cast<long long>(el * pt.size + pt.rank) * p.cap + ps) * p.H);
                ws[s] = p.w ? p.w[t * p.k + s] : 1.f;
            }
        }
    }
    if (p.dw) {
        // gradient of the combine weights: dw[t, s] = <dot_with[t], expert_output(t, s)>
        float acc[kMoeMaxK];
#pragma unroll
        for (int s = 0; s < kMoeMaxK; ++s) acc[s] = 0.f;
        const uint4* d = reinterpret_cast<const uint4*>(p.dot_with + t * p.H);
        for (int c = lane; c < hv; c += 32) {
            float df[8];
            unpack8(d[c], df);
#pragma unroll
            for (int s = 0; s < kMoeMaxK; ++s)
                if (rows[s]) {
                    float f[8];
                    unpack8(rows[s][c], f);
#pragma unroll
                    for (int q = 0; q < 8; ++q) acc[s] += f[q] * df[q];
                }
        }
#pragma unroll
        for (int s = 0; s < kMoeMaxK; ++s) {
            const float v = warp_sum(acc[s]);
            if (lane == 0 && s < p.k) p.dw[t * p.k + s] = v;
        }
        return;
    }
    const uint4* b = p.base ? reinterpret_cast<const uint4*>(p.base + t * p.H) : nullptr;
    uint4* o = reinterpret_cast<uint4*>(p.out + t * p.H);
    for (int c = lane; c < hv; c += 32) {
        uint4 v[kMoeMaxK];
#pragma unroll
        for (int s = 0; s < kMoeMaxK; ++s)
            if (rows[s]) v[s] = rows[s][c];
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (b) unpack8(b[c], acc);
#pragma unroll
        for (int s = 0; s < kMoeMaxK; ++s)
            if (rows[s]) {
                float f[8];
                unpack8(v[s], f);
#pragma unroll
                for (int q = 0; q < 8; ++q) acc[q] += ws[s] * f[q];
            }
        o[c] = pack8(acc);
    }
}

}  // namespace cai

using namespace cai;

CAI_API int cai_moe_route_fwd(const float* logits, int* idx, float* w, int* pos, int* counts, int T, int E, int k, int cap,
                              void* stream) {
    if (E % 32 || E > 32 * kMoeMaxEPerLane || k < 1 || k > kMoeMaxK || k > E) {
        set_last_error("moe_route: experts must be a multiple of 32 (<= 256) and top_k <= 8");
        return CAI_K_BAD_ARG;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    moe_route_fwd_kernel<<<(T * 32 + 255) / 256, 256, 0, st>>>(logits, idx, w, pos, counts, T, E, k, cap);
    moe_assign_slots_kernel<<<E, 256, 0, st>>>(idx, pos, counts, T * k, cap);
    return cudaGetLastError() == cudaSuccess ? 0 : CAI_K_CUDA;
}

CAI_API int cai_moe_route_bwd(const float* logits, const int* idx, const float* dw, const int* pos, void* dlogits, int T, int E,
                              int k, void* stream) {
    moe_route_bwd_kernel<<<(T * 32 + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        logits, idx, dw, pos, static_cast<__nv_bfloat16*>(dlogits), T, E, k);
    return cudaGetLastError() == cudaSuccess ? 0 : CAI_K_CUDA;
}

int cai_moe_dispatch(const PeerTable& pt, const void* rows, const int* idx, const int* pos, const float* scale,
                     const int* counts, unsigned long long slab_off, unsigned long long cnt_off, int T, int H, int k, int E,
                     int cap, const uint32_t* epoch_base, uint32_t seq, unsigned int* done_counter, cudaStream_t st) {
    if ((H & 7) || E % pt.size || cap % 128) {
        set_last_error("moe_dispatch: H %% 8, experts %% group size and capacity %% 128 must be 0");
        return CAI_K_BAD_ARG;
    }
    MoeDispatchParams p;
    p.rows = static_cast<const __nv_bfloat16*>(rows);
    p.idx = idx; p.pos = pos; p.scale = scale; p.counts = counts;
    p.slab_off = slab_off; p.cnt_off = cnt_off;
    p.T = T; p.H = H; p.k = k; p.E = E; p.E_l = E / pt.size; p.cap = cap;
    p.epoch_base = epoch_base; p.seq = seq; p.done_counter = done_counter;
    const int dev = current_device();
    p.status = status_words(dev);
    const int grid = sm_count(dev) * 4;
    moe_dispatch_kernel<<<grid, 256, 0, st>>>(pt, p);
    return cudaGetLastError() == cudaSuccess ? 0 : CAI_K_CUDA;
}

int cai_moe_combine(const PeerTable& pt, const void* base, void* out, const int* idx, const int* pos, const float* w,
                    unsigned long long slab_off, const void* dot_with, float* dw, int T, int H, int k, int E, int cap,
                    int announce, const uint32_t* epoch_base, uint32_t seq, cudaStream_t st) {
    MoeCombineParams p;
    p.base = static_cast<const __nv_bfloat16*>(base);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.idx = idx; p.pos = pos; p.w = w;
    p.slab_off = slab_off;
    p.dot_with = static_cast<const __nv_bfloat16*>(dot_with);
    p.dw = dw;
    p.T = T; p.H = H; p.k = k; p.E_l = E / pt.size; p.cap = cap;
    p.announce = announce;
    p.epoch_base = epoch_base; p.seq = seq;
    p.status = status_words(current_device());
    moe_combine_kernel<<<(static_cast<long long>(T) * 32 + 255) / 256, 256, 0, st>>>(pt, p);
    return cudaGetLastError() == cudaSuccess ? 0 : CAI_K_CUDA;
}

CAI_API unsigned long long cai_signal_block_bytes(void) { return kSigBytes; }

static PeerTable table_of(void* const* bases, int rank, int size, unsigned long long sig_off) {
    PeerTable pt{};
    for (int i = 0; i < size && i < kMaxPeers; ++i) pt.base[i] = static_cast<uint8_t*>(bases[i]);
    pt.rank = rank;
    pt.size = size;
    pt.sig_off = sig_off;
    return pt;
}

CAI_API int cai_moe_dispatch_c(void* const* bases, int rank, int size, unsigned long long sig_off, const void* rows,
                               const int* idx, const int* pos, const float* scale, const int* counts,
                               unsigned long long slab_off, unsigned long long cnt_off, int T, int H, int k, int E, int cap,
                               const uint32_t* epoch_base, uint32_t seq, unsigned int* scratch, void* stream) {
    if (size < 1 || size > kMaxPeers) return CAI_K_BAD_ARG;
    return cai_moe_dispatch(table_of(bases, rank, size, sig_off), rows, idx, pos, scale, counts, slab_off, cnt_off, T, H, k, E,
                            cap, epoch_base, seq, scratch, static_cast<cudaStream_t>(stream));
}

CAI_API int cai_moe_combine_c(void* const* bases, int rank, int size, unsigned long long sig_off, const void* base, void* out,
                              const int* idx, const int* pos, const float* w, unsigned long long slab_off, const void* dot_with,
                              float* dw, int T, int H, int k, int E, int cap, int announce, const uint32_t* epoch_base,
                              uint32_t seq, void* stream) {
    if (size < 1 || size > kMaxPeers) return CAI_K_BAD_ARG;
    return cai_moe_combine(table_of(bases, rank, size, sig_off), base, out, idx, pos, w, slab_off, dot_with, dw, T, H, k, E, cap,
                           announce, epoch_base, seq, static_cast<cudaStream_t>(stream));
}
