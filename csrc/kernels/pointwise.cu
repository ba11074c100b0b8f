// pointwise.cu - bandwidth-bound kernels: RMSNorm fwd/bwd, rotary embedding, SwiGLU fwd/bwd,
// embedding gather / scatter-add, fused softmax cross-entropy, AdamW, casts.
//
// All of them stream bf16 rows with 16-byte vector accesses and keep reductions in fp32.
// They replace the scalar one-element-per-thread fp32 kernels of the reference
// (src/cuda/cai_kernels.cu) and fix two of its defects on the way: rmsnorm backward can
// accumulate into dx (the residual path, src/refmodel.c:453,467), and the rotary embedding is
// real rather than a placeholder (src/cuda/cai_kernels.cu:216-220).
#include <math.h>

#include "cai_kernels.h"
#include "host_common.h"
#include "norm_kernels.cuh"
#include "sm100.cuh"

namespace cai {

#define CAI_LAUNCH_CHECK(name)                                                          \
    do {                                                                                \
        cudaError_t e__ = cudaGetLastError();                                           \
        if (e__ != cudaSuccess) {                                                       \
            set_last_error("%s launch failed: %s", name, cudaGetErrorString(e__));      \
            return CAI_K_CUDA;                                                          \
        }                                                                               \
    } while (0)

// ------------------------------------------------------------------ RMSNorm
// A row is handled by R = ceil(H / 2048) warps, each lane keeping 64 elements of x (and dy) in
// registers, so every tensor is read exactly once and no block-wide barrier sits between the
// reduction and the second sweep when R = 1. A CTA of 8 warps works on 8 / R rows at a time.
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows, int H, float eps, int R) {
    __shared__ float part[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = 8 / R;
    const int grp = warp / R, sub = warp - grp * R;
    const bool active = grp < groups;
    const int col0 = sub * kNormWarpCols;
    const uint4* gr = reinterpret_cast<const uint4*>(g);
    for (long long base = static_cast<long long>(blockIdx.x) * groups; base < rows; base += static_cast<long long>(gridDim.x) * groups) {
        const long long row = base + grp;
        const bool live = active && row < rows;
        uint4 xv[8];
        float ss = 0.f;
        if (live) {
            const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int col = col0 + (c * 32 + lane) * 8;
                if (col < H) {
                    xv[c] = xr[col >> 3];
                    float f[8];
                    unpack8(xv[c], f);
#pragma unroll
                    for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
                }
            }
        }
        ss = warp_sum(ss);
        if (R > 1) {
            if (lane == 0) part[warp] = ss;
            __syncthreads();
            if (active) {
                ss = 0.f;
                for (int k = 0; k < R; ++k) ss += part[grp * R + k];
            }
            __syncthreads();
        }
        if (live) {
            const float rr = rsqrtf(ss / H + eps);
            if (sub == 0 && lane == 0 && rstd) rstd[row] = rr;
            uint4* yr = reinterpret_cast<uint4*>(y + row * H);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int col = col0 + (c * 32 + lane) * 8;
                if (col < H) {
                    float f[8], gg[8];
                    unpack8(xv[c], f);
                    unpack8(gr[col >> 3], gg);
#pragma unroll
                    for (int e = 0; e < 8; ++e) f[e] = f[e] * rr * gg[e];
                    yr[col >> 3] = pack8(f);
                }
            }
        }
    }
}

// ------------------------------------------------------------------ rotary embedding
__global__ void rope_table_kernel(float2* table, int seq, int half, float theta) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= seq * half) return;
    const int pos = idx / half, i = idx % half;
    const float inv_freq = powf(theta, -static_cast<float>(i) / static_cast<float>(half));
    float s, c;
    sincosf(static_cast<float>(pos) * inv_freq, &s, &c);
    table[idx] = make_float2(c, s);
}

// One thread rotates 8 pairs (i .. i+7, i+half .. i+half+7) of one head of one token.
__global__ void rope_apply_kernel(__nv_bfloat16* qkv, const float2* __restrict__ table, long long T, int seq,
                                  int nh, int nkv, int hd, long long ld, int inverse) {
    const int half = hd >> 1;
    const int per_head = half >> 3;
    const int heads = nh + nkv;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = T * heads * per_head;
    if (idx >= total) return;
    const int v = idx % per_head;
    const int head = (idx / per_head) % heads;
    const long long t = idx / ((long long)per_head * heads);
    const int pos = t % seq;
    __nv_bfloat16* base = qkv + t * ld + (long long)head * hd + v * 8;
    const float2* tb = table + (long long)pos * half + v * 8;
    float a[8], b[8];
    unpack8(*reinterpret_cast<const uint4*>(base), a);
    unpack8(*reinterpret_cast<const uint4*>(base + half), b);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float2 cs = tb[e];
        const float sn = inverse ? -cs.y : cs.y;
        const float x1 = a[e] * cs.x - b[e] * sn;
        const float x2 = b[e] * cs.x + a[e] * sn;
        a[e] = x1;
        b[e] = x2;
    }
    *reinterpret_cast<uint4*>(base) = pack8(a);
    *reinterpret_cast<uint4*>(base + half) = pack8(b);
}

// ------------------------------------------------------------------ SwiGLU
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act,
                                  long long T, int F) {
    const int fv = F >> 3;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * fv) return;
    const long long t = idx / fv;
    const int c = idx % fv;
    const __nv_bfloat16* row = gu + t * 2 * F;
    float g[8], u[8];
    unpack8(*reinterpret_cast<const uint4*>(row + c * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(row + F + c * 8), u);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float s = 1.f / (1.f + __expf(-g[e]));
        g[e] = g[e] * s * u[e];
    }
    *reinterpret_cast<uint4*>(act + t * F + c * 8) = pack8(g);
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int F) {
    const int fv = F >> 3;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * fv) return;
    const long long t = idx / fv;
    const int c = idx % fv;
    const __nv_bfloat16* row = gu + t * 2 * F;
    float g[8], u[8], d[8];
    unpack8(*reinterpret_cast<const uint4*>(row + c * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(row + F + c * 8), u);
    unpack8(*reinterpret_cast<const uint4*>(dact + t * F + c * 8), d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float s = 1.f / (1.f + __expf(-g[e]));
        const float silu = g[e] * s;
        const float dg = d[e] * u[e] * s * (1.f + g[e] * (1.f - s));
        const float du = d[e] * silu;
        g[e] = dg;
        u[e] = du;
    }
    __nv_bfloat16* orow = dgu + t * 2 * F;
    *reinterpret_cast<uint4*>(orow + c * 8) = pack8(g);
    *reinterpret_cast<uint4*>(orow + F + c * 8) = pack8(u);
}

// ------------------------------------------------------------------ embedding
__global__ void embed_fwd_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ E,
                                 __nv_bfloat16* __restrict__ out, int H, int lo, int hi) {
    const long long t = blockIdx.x;
    const int tok = tokens[t];
    const int nv = H >> 3;
    uint4* o = reinterpret_cast<uint4*>(out + t * H);
    if (tok < lo || tok >= hi) {
        for (int i = threadIdx.x; i < nv; i += blockDim.x) o[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    const uint4* e = reinterpret_cast<const uint4*>(E + (long long)(tok - lo) * H);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) o[i] = e[i];
}

// Embedding backward without atomics: a CTA owns kEmbRows consecutive vocabulary rows, scans the token list front to
// back and adds the gradient row of every token that falls into its range, in token order. Each row of dE has one
// writer and a fixed order of additions, so the result is the same in every run (the reference scatters with
// atomicAdd, src/cuda/cai_kernels.cu:26-34).
constexpr int kEmbRows = 32;
__global__ void __launch_bounds__(256)
embed_bwd_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ dout, float* __restrict__ dE, int T, int H,
                 int lo, int hi) {
    __shared__ unsigned match[8];
    __shared__ int toks[256];
    const int v0 = lo + static_cast<int>(blockIdx.x) * kEmbRows;
    const int v1 = v0 + kEmbRows < hi ? v0 + kEmbRows : hi;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t0 = 0; t0 < T; t0 += 256) {
        const int t = t0 + threadIdx.x;
        const int tok = t < T ? tokens[t] : -1;
        const unsigned m = __ballot_sync(0xffffffffu, tok >= v0 && tok < v1);
        toks[threadIdx.x] = tok;
        if (lane == 0) match[warp] = m;
        __syncthreads();
        for (int w = 0; w < 8; ++w) {
            unsigned bits = match[w];
            while (bits) {
                const int b = __ffs(bits) - 1;
                bits &= bits - 1;
                const int tt = t0 + w * 32 + b;
                float* row = dE + static_cast<long long>(toks[w * 32 + b] - lo) * H;
                const __nv_bfloat16* d = dout + static_cast<long long>(tt) * H;
                for (int i = threadIdx.x; i < H; i += 256) row[i] += __bfloat162float(d[i]);
            }
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------ cross entropy
// One CTA per row: online (max, sum-exp) over the row, then a second sweep that overwrites the
// logits with (softmax - onehot) * grad_scale. The second sweep re-reads a row this CTA just
// streamed, so it is served from L2.
constexpr int kCeThreads = 512;
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_kernel(__nv_bfloat16* logits, const int* __restrict__ targets, float* loss_sum, float* row_lse,
                     int V, long long ld, float grad_scale, float loss_scale) {
    __shared__ float red[33];
    const long long row = blockIdx.x;
    __nv_bfloat16* lr = logits + row * ld;
    uint4* l4 = reinterpret_cast<uint4*>(lr);
    const int nv = V >> 3;
    const int tgt = targets[row];
    float mx = -INFINITY, sum = 0.f;
    for (int i = threadIdx.x; i < nv; i += kCeThreads) {
        float f[8];
        unpack8(l4[i], f);
        float m8 = f[0];
#pragma unroll
        for (int e = 1; e < 8; ++e) m8 = fmaxf(m8, f[e]);
        if (m8 > mx) {
            sum *= __expf(mx - m8);
            mx = m8;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += __expf(f[e] - mx);
    }
    const float gmx = block_max(mx, red);
    sum *= (mx == -INFINITY) ? 0.f : __expf(mx - gmx);
    const float gsum = block_sum(sum, red);
    const float lse = gmx + logf(gsum);
    if (threadIdx.x == 0) {
        if (row_lse) row_lse[row] = lse;
        if (tgt >= 0 && tgt < V && loss_sum)
            atomicAdd(loss_sum, (lse - __bfloat162float(lr[tgt])) * loss_scale);
    }
    __syncthreads();
    const float gs = (tgt >= 0) ? grad_scale : 0.f;
    for (int i = threadIdx.x; i < nv; i += kCeThreads) {
        float f[8];
        unpack8(l4[i], f);
        const int c0 = i * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float p = __expf(f[e] - lse);
            if (c0 + e == tgt) p -= 1.f;
            f[e] = p * gs;
        }
        l4[i] = pack8(f);
    }
}

// Vocabulary-parallel variant: every rank holds V_local columns of the logits. Row maxima and
// exp-sums are reduced over the tensor-parallel group between the three kernels.
__global__ void __launch_bounds__(kCeThreads)
ce_rowmax_kernel(const __nv_bfloat16* __restrict__ logits, float* __restrict__ rowmax, int V, long long ld) {
    __shared__ float red[33];
    const long long row = blockIdx.x;
    const uint4* l4 = reinterpret_cast<const uint4*>(logits + row * ld);
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < (V >> 3); i += kCeThreads) {
        float f[8];
        unpack8(l4[i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) mx = fmaxf(mx, f[e]);
    }
    mx = block_max(mx, red);
    if (threadIdx.x == 0) rowmax[row] = mx;
}
__global__ void __launch_bounds__(kCeThreads)
ce_rowsum_kernel(const __nv_bfloat16* __restrict__ logits, const float* __restrict__ rowmax,
                 float* __restrict__ rowsum, int V, long long ld) {
    __shared__ float red[33];
    const long long row = blockIdx.x;
    const uint4* l4 = reinterpret_cast<const uint4*>(logits + row * ld);
    const float mx = rowmax[row];
    float sum = 0.f;
    for (int i = threadIdx.x; i < (V >> 3); i += kCeThreads) {
        float f[8];
        unpack8(l4[i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += __expf(f[e] - mx);
    }
    sum = block_sum(sum, red);
    if (threadIdx.x == 0) rowsum[row] = sum;
}
__global__ void __launch_bounds__(kCeThreads)
ce_grad_tp_kernel(__nv_bfloat16* logits, const int* __restrict__ targets, const float* __restrict__ rowmax,
                  const float* __restrict__ rowsum, float* loss_sum, int V, long long ld, int vocab_lo,
                  int add_lse, float grad_scale, float loss_scale) {
    const long long row = blockIdx.x;
    __nv_bfloat16* lr = logits + row * ld;
    uint4* l4 = reinterpret_cast<uint4*>(lr);
    const int tgt_global = targets[row];
    const int tgt = tgt_global - vocab_lo;  // local column, may be out of range
    const float lse = rowmax[row] + logf(rowsum[row]);
    if (threadIdx.x == 0 && loss_sum && tgt_global >= 0) {
        float contrib = add_lse ? lse : 0.f;
        if (tgt >= 0 && tgt < V) contrib -= __bfloat162float(lr[tgt]);
        atomicAdd(loss_sum, contrib * loss_scale);
    }
    __syncthreads();
    const float gs = tgt_global >= 0 ? grad_scale : 0.f;
    for (int i = threadIdx.x; i < (V >> 3); i += kCeThreads) {
        float f[8];
        unpack8(l4[i], f);
        const int c0 = i * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float p = __expf(f[e] - lse);
            if (c0 + e == tgt) p -= 1.f;
            f[e] = p * gs;
        }
        l4[i] = pack8(f);
    }
}

// ------------------------------------------------------------------ AdamW
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ grad, __nv_bfloat16* __restrict__ param, long long n,
                             float lr, float b1, float b2, float eps, float wd, float gscale, float bc1,
                             float bc2) {
    const long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i4 >= n) return;
    if (i4 + 4 <= n) {
        float4 p = *reinterpret_cast<float4*>(master + i4);
        float4 mm = *reinterpret_cast<float4*>(m + i4);
        float4 vv = *reinterpret_cast<float4*>(v + i4);
        const float4 g = *reinterpret_cast<const float4*>(grad + i4);
        float pa[4] = {p.x, p.y, p.z, p.w}, ma[4] = {mm.x, mm.y, mm.z, mm.w}, va[4] = {vv.x, vv.y, vv.z, vv.w};
        const float ga[4] = {g.x * gscale, g.y * gscale, g.z * gscale, g.w * gscale};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            ma[e] = b1 * ma[e] + (1.f - b1) * ga[e];
            va[e] = b2 * va[e] + (1.f - b2) * ga[e] * ga[e];
            const float mh = ma[e] / bc1, vh = va[e] / bc2;
            pa[e] -= lr * (mh / (sqrtf(vh) + eps) + wd * pa[e]);
        }
        *reinterpret_cast<float4*>(master + i4) = make_float4(pa[0], pa[1], pa[2], pa[3]);
        *reinterpret_cast<float4*>(m + i4) = make_float4(ma[0], ma[1], ma[2], ma[3]);
        *reinterpret_cast<float4*>(v + i4) = make_float4(va[0], va[1], va[2], va[3]);
        if (param) {
            uint2 o;
            o.x = pack_bf16(pa[0], pa[1]);
            o.y = pack_bf16(pa[2], pa[3]);
            *reinterpret_cast<uint2*>(param + i4) = o;
        }
    } else {
        for (long long i = i4; i < n; ++i) {
            const float g = grad[i] * gscale;
            const float mn = b1 * m[i] + (1.f - b1) * g;
            const float vn = b2 * v[i] + (1.f - b2) * g * g;
            float p = master[i];
            p -= lr * ((mn / bc1) / (sqrtf(vn / bc2) + eps) + wd * p);
            m[i] = mn;
            v[i] = vn;
            master[i] = p;
            if (param) param[i] = __float2bfloat16(p);
        }
    }
}

// ------------------------------------------------------------------ utilities
__global__ void cast_f32_bf16_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ d, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) d[i] = __float2bfloat16(s[i]);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ s, float* __restrict__ d, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) d[i] = __bfloat162float(s[i]);
}
__global__ void fill_f32_kernel(float* d, float v, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) d[i] = v;
}
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ o, long long n8) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    float x[8], y[8];
    unpack8(reinterpret_cast<const uint4*>(a)[i], x);
    unpack8(reinterpret_cast<const uint4*>(b)[i], y);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] += y[e];
    reinterpret_cast<uint4*>(o)[i] = pack8(x);
}

static inline unsigned blocks_for(long long n, int threads) {
    return static_cast<unsigned>((n + threads - 1) / threads);
}

}  // namespace cai

using namespace cai;

static int norm_row_warps(int H) { return (H + kNormWarpCols - 1) / kNormWarpCols; }

CAI_API int cai_rmsnorm_fwd(const void* x, const void* g, void* y, float* rstd, int rows, int H, float eps,
                            void* stream) {
    if (rows <= 0) return CAI_K_OK;
    const int R = norm_row_warps(H);
    if ((H & 7) || R > 8) {
        set_last_error("rmsnorm: H must be a multiple of 8 and <= 16384");
        return CAI_K_BAD_ARG;
    }
    const int groups = 8 / R;
    const long long want = (static_cast<long long>(rows) + groups - 1) / groups;
    const int cap = cai_rmsnorm_bwd_parts(rows) * 4;
    const int grid = static_cast<int>(want < cap ? want : cap);
    rmsnorm_fwd_kernel<<<grid, kNormThreads, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)g,
                                                                       (__nv_bfloat16*)y, rstd, rows, H, eps, R);
    CAI_LAUNCH_CHECK("rmsnorm_fwd");
    return CAI_K_OK;
}

// Number of [H]-float partial rows cai_rmsnorm_bwd writes into its scratch buffer.
CAI_API int cai_rmsnorm_bwd_parts(int rows) {
    int sms = sm_count(current_device());
    if (sms <= 0) sms = 148;
    const int cap = sms * 2;
    return rows < cap ? rows : cap;
}

CAI_API int cai_rmsnorm_bwd(const void* x, const void* g, const float* rstd, const void* dy, void* dx, float* dg,
                            float* dg_partial, int rows, int H, int dx_accumulate, int dg_accumulate,
                            void* stream) {
    if (rows <= 0) return CAI_K_OK;
    const int R = norm_row_warps(H);
    if ((H & 7) || R > 8) {
        set_last_error("rmsnorm_bwd: H must be a multiple of 8 and <= 16384");
        return CAI_K_BAD_ARG;
    }
    if (launch_rmsnorm_bwd(x, g, rstd, dy, dx, dg, dg_partial, cai_rmsnorm_bwd_parts(rows), sm_count(current_device()), rows,
                           H, dx_accumulate, dg_accumulate, (cudaStream_t)stream) != 0) {
        set_last_error("rmsnorm_bwd launch failed");
        return CAI_K_CUDA;
    }
    return CAI_K_OK;
}

CAI_API int cai_rope_table(float* table, int seq, int hd, float theta, void* stream) {
    const int half = hd / 2;
    rope_table_kernel<<<blocks_for((long long)seq * half, 256), 256, 0, (cudaStream_t)stream>>>(
        (float2*)table, seq, half, theta);
    CAI_LAUNCH_CHECK("rope_table");
    return CAI_K_OK;
}

CAI_API int cai_rope_apply(void* qkv, const float* table, int T, int seq, int nh, int nkv, int hd, long long ld,
                           int inverse, void* stream) {
    if (T <= 0) return CAI_K_OK;
    if ((hd & 15) || (ld & 7)) {
        set_last_error("rope: head_dim must be a multiple of 16 and ld of 8");
        return CAI_K_BAD_ARG;
    }
    const long long total = (long long)T * (nh + nkv) * (hd / 16);
    rope_apply_kernel<<<blocks_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
        (__nv_bfloat16*)qkv, (const float2*)table, T, seq, nh, nkv, hd, ld, inverse);
    CAI_LAUNCH_CHECK("rope_apply");
    return CAI_K_OK;
}

CAI_API int cai_swiglu_fwd(const void* gu, void* act, int T, int F, void* stream) {
    if (T <= 0) return CAI_K_OK;
    if (F & 7) {
        set_last_error("swiglu: F must be a multiple of 8");
        return CAI_K_BAD_ARG;
    }
    swiglu_fwd_kernel<<<blocks_for((long long)T * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)gu, (__nv_bfloat16*)act, T, F);
    CAI_LAUNCH_CHECK("swiglu_fwd");
    return CAI_K_OK;
}

CAI_API int cai_swiglu_bwd(const void* gu, const void* dact, void* dgu, int T, int F, void* stream) {
    if (T <= 0) return CAI_K_OK;
    if (F & 7) {
        set_last_error("swiglu: F must be a multiple of 8");
        return CAI_K_BAD_ARG;
    }
    swiglu_bwd_kernel<<<blocks_for((long long)T * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dact, (__nv_bfloat16*)dgu, T, F);
    CAI_LAUNCH_CHECK("swiglu_bwd");
    return CAI_K_OK;
}

CAI_API int cai_embed_fwd(const int* tokens, const void* E, void* out, int T, int H, int vocab_lo, int vocab_hi,
                          void* stream) {
    if (T <= 0) return CAI_K_OK;
    if (H & 7) {
        set_last_error("embed: H must be a multiple of 8");
        return CAI_K_BAD_ARG;
    }
    embed_fwd_kernel<<<T, 128, 0, (cudaStream_t)stream>>>(tokens, (const __nv_bfloat16*)E, (__nv_bfloat16*)out, H,
                                                          vocab_lo, vocab_hi);
    CAI_LAUNCH_CHECK("embed_fwd");
    return CAI_K_OK;
}

CAI_API int cai_embed_bwd(const int* tokens, const void* dout, float* dE, int T, int H, int vocab_lo,
                          int vocab_hi, void* stream) {
    if (T <= 0) return CAI_K_OK;
    if (vocab_hi <= vocab_lo) return CAI_K_OK;
    embed_bwd_kernel<<<(vocab_hi - vocab_lo + kEmbRows - 1) / kEmbRows, 256, 0, (cudaStream_t)stream>>>(
        tokens, (const __nv_bfloat16*)dout, dE, T, H, vocab_lo, vocab_hi);
    CAI_LAUNCH_CHECK("embed_bwd");
    return CAI_K_OK;
}

CAI_API int cai_cross_entropy(void* logits, const int* targets, float* loss_sum, float* row_lse, int rows, int V,
                              long long ld, float grad_scale, float loss_scale, void* stream) {
    if (rows <= 0) return CAI_K_OK;
    if ((V & 7) || (ld & 7)) {
        set_last_error("cross_entropy: V and ld must be multiples of 8");
        return CAI_K_BAD_ARG;
    }
    cross_entropy_kernel<<<rows, kCeThreads, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, targets, loss_sum,
                                                                        row_lse, V, ld, grad_scale, loss_scale);
    CAI_LAUNCH_CHECK("cross_entropy");
    return CAI_K_OK;
}

CAI_API int cai_ce_rowmax(const void* logits, float* rowmax, int rows, int V, long long ld, void* stream) {
    if (rows <= 0) return CAI_K_OK;
    ce_rowmax_kernel<<<rows, kCeThreads, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, rowmax, V, ld);
    CAI_LAUNCH_CHECK("ce_rowmax");
    return CAI_K_OK;
}
CAI_API int cai_ce_rowsum(const void* logits, const float* rowmax, float* rowsum, int rows, int V, long long ld,
                          void* stream) {
    if (rows <= 0) return CAI_K_OK;
    ce_rowsum_kernel<<<rows, kCeThreads, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, rowmax, rowsum, V, ld);
    CAI_LAUNCH_CHECK("ce_rowsum");
    return CAI_K_OK;
}
CAI_API int cai_ce_grad_tp(void* logits, const int* targets, const float* rowmax, const float* rowsum, float* loss_sum,
                           int rows, int V, long long ld, int vocab_lo, int add_lse, float grad_scale, float loss_scale,
                           void* stream) {
    if (rows <= 0) return CAI_K_OK;
    ce_grad_tp_kernel<<<rows, kCeThreads, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, targets, rowmax, rowsum,
                                                                     loss_sum, V, ld, vocab_lo, add_lse, grad_scale,
                                                                     loss_scale);
    CAI_LAUNCH_CHECK("ce_grad_tp");
    return CAI_K_OK;
}

CAI_API int cai_adamw(float* master, float* m, float* v, const float* grad, void* param_bf16, long long n,
                      float lr, float beta1, float beta2, float eps, float wd, float grad_scale, int step,
                      void* stream) {
    if (n <= 0) return CAI_K_OK;
    const float bc1 = 1.f - powf(beta1, (float)step);
    const float bc2 = 1.f - powf(beta2, (float)step);
    adamw_kernel<<<blocks_for((n + 3) / 4, 256), 256, 0, (cudaStream_t)stream>>>(
        master, m, v, grad, (__nv_bfloat16*)param_bf16, n, lr, beta1, beta2, eps, wd, grad_scale, bc1, bc2);
    CAI_LAUNCH_CHECK("adamw");
    return CAI_K_OK;
}

CAI_API int cai_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream) {
    if (n <= 0) return CAI_K_OK;
    cast_f32_bf16_kernel<<<blocks_for(n, 256), 256, 0, (cudaStream_t)stream>>>(src, (__nv_bfloat16*)dst, n);
    CAI_LAUNCH_CHECK("cast_f32_bf16");
    return CAI_K_OK;
}
CAI_API int cai_cast_bf16_to_f32(const void* src, float* dst, long long n, void* stream) {
    if (n <= 0) return CAI_K_OK;
    cast_bf16_f32_kernel<<<blocks_for(n, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, dst, n);
    CAI_LAUNCH_CHECK("cast_bf16_f32");
    return CAI_K_OK;
}
CAI_API int cai_fill_f32(float* dst, float v, long long n, void* stream) {
    if (n <= 0) return CAI_K_OK;
    fill_f32_kernel<<<blocks_for(n, 256), 256, 0, (cudaStream_t)stream>>>(dst, v, n);
    CAI_LAUNCH_CHECK("fill_f32");
    return CAI_K_OK;
}
CAI_API int cai_add_bf16(const void* a, const void* b, void* out, long long n, void* stream) {
    if (n <= 0) return CAI_K_OK;
    if (n & 7) {
        set_last_error("add_bf16: n must be a multiple of 8");
        return CAI_K_BAD_ARG;
    }
    add_bf16_kernel<<<blocks_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, n / 8);
    CAI_LAUNCH_CHECK("add_bf16");
    return CAI_K_OK;
}
CAI_API int cai_l2_flush(void* scratch, long long bytes, void* stream) {
    return cudaMemsetAsync(scratch, 0, (size_t)bytes, (cudaStream_t)stream) == cudaSuccess ? CAI_K_OK : CAI_K_CUDA;
}
