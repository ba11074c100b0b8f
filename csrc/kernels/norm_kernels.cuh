// norm_kernels.cuh - device code of RMSNorm backward, shared by the two translation units that
// launch it (pointwise.cu and rmsnorm_bwd_static.cu), plus the small vector / reduction helpers the
// bandwidth-bound kernels use. Kernels are `static` so that each including file owns its copy.
#pragma once

#include <math.h>

#include "sm100.cuh"

namespace cai {

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x);
    f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z);
    f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 o;
    o.x = pack_bf16(f[0], f[1]);
    o.y = pack_bf16(f[2], f[3]);
    o.z = pack_bf16(f[4], f[5]);
    o.w = pack_bf16(f[6], f[7]);
    return o;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over the block; every thread gets the result. `red` is >= 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

constexpr int kNormThreads = 256;
constexpr int kNormWarpCols = 2048;  // columns one warp covers: 32 lanes x 8 chunks x 8 elements

// Backward, input gradient: dx (+)= rr * dy * g - rr^3 * x * sum(dy * g * x) / H. A row is handled
// by R = ceil(H / 2048) warps that keep their slice of x and dy in registers (each tensor is read
// once); a CTA of 8 warps works on 8 / R rows at a time.
static __global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                      const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dy,
                      __nv_bfloat16* __restrict__ dx, int rows, int H, int dx_acc, int R) {
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
        uint4 xv[8], dv[8];
        float S = 0.f;
        if (live) {
            const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
            const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * H);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int col = col0 + (c * 32 + lane) * 8;
                if (col < H) {
                    xv[c] = xr[col >> 3];
                    dv[c] = dyr[col >> 3];
                }
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int col = col0 + (c * 32 + lane) * 8;
                if (col < H) {
                    float xf[8], df[8], gf[8];
                    unpack8(xv[c], xf);
                    unpack8(dv[c], df);
                    unpack8(gr[col >> 3], gf);
#pragma unroll
                    for (int e = 0; e < 8; ++e) S += df[e] * gf[e] * xf[e];
                }
            }
        }
        S = warp_sum(S);
        if (R > 1) {
            if (lane == 0) part[warp] = S;
            __syncthreads();
            if (active) {
                S = 0.f;
                for (int k = 0; k < R; ++k) S += part[grp * R + k];
            }
            __syncthreads();
        }
        if (live) {
            const float rr = rstd[row];
            const float k3 = rr * rr * rr * S / H;
            uint4* dxr = reinterpret_cast<uint4*>(dx + row * H);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int col = col0 + (c * 32 + lane) * 8;
                if (col < H) {
                    float xf[8], df[8], gf[8], o[8];
                    unpack8(xv[c], xf);
                    unpack8(dv[c], df);
                    unpack8(gr[col >> 3], gf);
                    if (dx_acc) unpack8(dxr[col >> 3], o);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float v = rr * df[e] * gf[e] - k3 * xf[e];
                        o[e] = dx_acc ? o[e] + v : v;
                    }
                    dxr[col >> 3] = pack8(o);
                }
            }
        }
    }
}

// Backward, gain gradient: partial[part][col] = sum over the part's rows of dy * x * rstd. Threads
// own columns (coalesced 16-byte loads), CTAs own row ranges; x and dy were just streamed by the dx
// kernel, so this second sweep is mostly served from L2.
static __global__ void __launch_bounds__(256)
rmsnorm_bwd_dg_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ rstd,
                      const __nv_bfloat16* __restrict__ dy, float* __restrict__ dg_partial, int rows, int H,
                      int rows_per_part) {
    const long long r0 = static_cast<long long>(blockIdx.x) * rows_per_part;
    const long long r1 = r0 + rows_per_part < rows ? r0 + rows_per_part : rows;
    for (int c = threadIdx.x; c < (H >> 3); c += 256) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (long long r = r0; r < r1; ++r) {
            float xf[8], df[8];
            unpack8(reinterpret_cast<const uint4*>(x + r * H)[c], xf);
            unpack8(reinterpret_cast<const uint4*>(dy + r * H)[c], df);
            const float rr = rstd[r];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += df[e] * xf[e] * rr;
        }
        float4* o = reinterpret_cast<float4*>(dg_partial + static_cast<long long>(blockIdx.x) * H + c * 8);
        o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
}

// out[col] (+)= sum over parts of parts[p][col]. A block covers 32 columns; its 8 warps split the
// partial rows, so a column's loads are spread over 8 independent chains instead of one long one.
static __global__ void __launch_bounds__(256)
reduce_parts_kernel(const float* __restrict__ parts, float* __restrict__ out, int nparts, int H, int accumulate) {
    __shared__ float acc[8][32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + lane;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (col < H) {
        int p = w;
        for (; p + 24 < nparts; p += 32) {
            s0 += parts[static_cast<long long>(p) * H + col];
            s1 += parts[static_cast<long long>(p + 8) * H + col];
            s2 += parts[static_cast<long long>(p + 16) * H + col];
            s3 += parts[static_cast<long long>(p + 24) * H + col];
        }
        for (; p < nparts; p += 8) s0 += parts[static_cast<long long>(p) * H + col];
    }
    acc[w][lane] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    if (w == 0 && col < H) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) s += acc[k][lane];
        out[col] = accumulate ? out[col] + s : s;
    }
}

// Backward in ONE sweep for H <= 8192: a row is handled by R = ceil(H / 1024) warps that keep their slice of x and
// dy in registers (32 elements per lane), write dx and add the row's dy * x * rstd into per-lane column sums that
// they carry across all the rows they handle; at the end the warps of a CTA combine their sums in shared memory
// (in a fixed order) and the CTA writes one partial row of the gain gradient. x and dy are read once (the
// two-kernel form above reads them twice). About 100 registers per thread, so two CTAs of eight warps share an SM
// and a CTA still fits beside a resident GEMM CTA of another stream.
constexpr int kNormFusedThreads = 256;
constexpr int kNormFusedCols = 1024;   // columns one warp covers: 32 lanes x 4 chunks x 8 elements
constexpr int kNormFusedMaxH = 8192;
static __global__ void __launch_bounds__(kNormFusedThreads, 2)
rmsnorm_bwd_fused_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                         const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dy,
                         __nv_bfloat16* __restrict__ dx, float* __restrict__ dg_partial, int rows, int H, int dx_acc, int R) {
    extern __shared__ float sdg[];   // H floats, then 8 partial row sums
    float* part = sdg + H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = 8 / R;                 // rows a CTA works on at a time
    const int grp = warp / R, sub = warp - grp * R;
    const bool active = grp < groups;
    const int col0 = sub * kNormFusedCols;
    const uint4* gr = reinterpret_cast<const uint4*>(g);
    for (int c = threadIdx.x; c < H; c += kNormFusedThreads) sdg[c] = 0.f;
    float acc[4][8];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[c][e] = 0.f;
    for (long long base = static_cast<long long>(blockIdx.x) * groups; base < rows; base += static_cast<long long>(gridDim.x) * groups) {
        const long long row = base + grp;
        const bool live = active && row < rows;
        uint4 xv[4], dv[4];
        float S = 0.f;
        if (live) {
            const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
            const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * H);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = col0 + (c * 32 + lane) * 8;
                if (col < H) {
                    xv[c] = xr[col >> 3];
                    dv[c] = dyr[col >> 3];
                }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = col0 + (c * 32 + lane) * 8;
                if (col < H) {
                    float xf[8], df[8], gf[8];
                    unpack8(xv[c], xf);
                    unpack8(dv[c], df);
                    unpack8(gr[col >> 3], gf);
#pragma unroll
                    for (int e = 0; e < 8; ++e) S += df[e] * gf[e] * xf[e];
                }
            }
        }
        S = warp_sum(S);
        if (R > 1) {
            if (lane == 0) part[warp] = S;
            __syncthreads();
            if (active) {
                S = 0.f;
                for (int k = 0; k < R; ++k) S += part[grp * R + k];
            }
            __syncthreads();
        }
        if (live) {
            const float rr = rstd[row];
            const float k3 = rr * rr * rr * S / H;
            uint4* dxr = reinterpret_cast<uint4*>(dx + row * H);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = col0 + (c * 32 + lane) * 8;
                if (col < H) {
                    float xf[8], df[8], gf[8], o[8];
                    unpack8(xv[c], xf);
                    unpack8(dv[c], df);
                    unpack8(gr[col >> 3], gf);
                    if (dx_acc) unpack8(dxr[col >> 3], o);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float v = rr * df[e] * gf[e] - k3 * xf[e];
                        o[e] = dx_acc ? o[e] + v : v;
                        acc[c][e] += df[e] * xf[e] * rr;
                    }
                    dxr[col >> 3] = pack8(o);
                }
            }
        }
    }
    // row groups take turns adding into the CTA's row (a fixed order, so the result does not depend on timing)
    __syncthreads();
    for (int w = 0; w < groups; ++w) {
        if (active && grp == w) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = col0 + (c * 32 + lane) * 8;
                if (col < H) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) sdg[col + e] += acc[c][e];
                }
            }
        }
        __syncthreads();
    }
    for (int c = threadIdx.x; c < H; c += kNormFusedThreads) dg_partial[static_cast<long long>(blockIdx.x) * H + c] = sdg[c];
}

// Host side of RMSNorm backward, shared by the entry points: `scratch` holds at most `parts_cap`
// rows of H floats. Returns a cudaError_t-style 0 / non-zero.
static inline int launch_rmsnorm_bwd(const void* x, const void* g, const float* rstd, const void* dy, void* dx, float* dg,
                                     float* scratch, int parts_cap, int sms, int rows, int H, int dx_accumulate,
                                     int dg_accumulate, cudaStream_t st) {
    if (H <= kNormFusedMaxH && (H & 7) == 0 && parts_cap >= 1) {
        // one sweep: dx and the partial gain gradients from the same read of x and dy
        int Rf = (H + kNormFusedCols - 1) / kNormFusedCols;
        Rf = Rf <= 1 ? 1 : Rf <= 2 ? 2 : Rf <= 4 ? 4 : 8;        // a divisor of the CTA's eight warps
        const int gpc = 8 / Rf;
        long long want = (static_cast<long long>(rows) + gpc - 1) / gpc;
        int grid = static_cast<int>(want < 2LL * sms ? want : 2LL * sms);
        if (grid > parts_cap) grid = parts_cap;
        if (grid < 1) grid = 1;
        const size_t smem = (static_cast<size_t>(H) + 8) * sizeof(float);
        rmsnorm_bwd_fused_kernel<<<grid, kNormFusedThreads, smem, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(g),
                                                                      rstd, static_cast<const __nv_bfloat16*>(dy),
                                                                      static_cast<__nv_bfloat16*>(dx), scratch, rows, H, dx_accumulate, Rf);
        reduce_parts_kernel<<<(H + 31) / 32, 256, 0, st>>>(scratch, dg, grid, H, dg_accumulate);
        return cudaGetLastError() == cudaSuccess ? 0 : 1;
    }
    const int R = (H + kNormWarpCols - 1) / kNormWarpCols;
    const int groups = 8 / R;
    const long long want = (static_cast<long long>(rows) + groups - 1) / groups;
    const int grid = static_cast<int>(want < sms * 8LL ? want : sms * 8LL);
    int parts = rows < parts_cap ? rows : parts_cap;
    const int rows_per_part = (rows + parts - 1) / parts;
    parts = (rows + rows_per_part - 1) / rows_per_part;
    rmsnorm_bwd_dg_kernel<<<parts, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rstd, static_cast<const __nv_bfloat16*>(dy),
                                                 scratch, rows, H, rows_per_part);
    reduce_parts_kernel<<<(H + 31) / 32, 256, 0, st>>>(scratch, dg, parts, H, dg_accumulate);
    // dx last: callers may pass dx == dy (in place), and the gain gradient needs the unmodified dy
    rmsnorm_bwd_dx_kernel<<<grid, kNormThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(g),
                                                        rstd, static_cast<const __nv_bfloat16*>(dy),
                                                        static_cast<__nv_bfloat16*>(dx), rows, H, dx_accumulate, R);
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

}  // namespace cai
