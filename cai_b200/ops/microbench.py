"""Micro-benchmarks of single kernels of the library (CUDA-event timed, L2 flushed between
iterations). Also the small fixed-size workloads that profiler captures are taken on.

    python -m cai_b200.ops.microbench gemm --m 8192 --n 8192 --k 8192 [--ta] [--tb] [--f32]
    python -m cai_b200.ops.microbench attn_fwd --batch 1 --seq 4096 --heads 16 --kv-heads 8
    python -m cai_b200.ops.microbench attn_bwd --batch 1 --seq 4096 --heads 16 --kv-heads 8
    python -m cai_b200.ops.microbench rmsnorm_bwd --rows 4096 --hidden 2048
    python -m cai_b200.ops.microbench swiglu --rows 4096 --ffn 8192
    python -m cai_b200.ops.microbench gemm_fp8 --m 8192 --n 8192 --k 8192
    python -m cai_b200.ops.microbench gemm_swiglu --m 8192 --n 16384 --k 2048     (n = 2 x ffn: gate and up)

Prints one JSON line per run: milliseconds (median of ``--iters`` after ``--warmup``), achieved
TFLOP/s or GB/s, and the fraction of the measured peaks in ``MEASURED_PEAKS.json`` when present.
"""
from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path

import torch

from . import (flash_attn_bwd, flash_attn_fwd, gemm, rmsnorm_bwd, rmsnorm_fwd, swiglu_bwd, swiglu_fwd)

ROOT = Path(__file__).resolve().parent.parent.parent


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


def timeit(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()          # write a buffer larger than L2 between timed iterations
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "gemm_fp8", "gemm_swiglu", "attn_fwd", "attn_bwd", "rmsnorm_bwd", "swiglu"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--ta", action="store_true")
    ap.add_argument("--tb", action="store_true")
    ap.add_argument("--f32", action="store_true", help="fp32 accumulate-into-C epilogue (weight-gradient form)")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--variant", type=int, default=0, help="attn_fwd: 0 auto, 1 one tile per CTA, 2 two tiles per CTA")
    ap.add_argument("--parts", type=int, default=7, help="attn_bwd: bit 0 delta, bit 1 dK/dV, bit 2 dQ")
    a = ap.parse_args(argv)
    dev = "cuda"
    bf = torch.bfloat16
    tf_peak, bw_peak, src = _peaks()
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = {"kernel": a.kernel}
    if a.kernel == "gemm":
        A = torch.randn((a.k, a.m) if a.ta else (a.m, a.k), device=dev, dtype=bf)
        B = torch.randn((a.k, a.n) if a.tb else (a.n, a.k), device=dev, dtype=bf)
        C = torch.zeros(a.m, a.n, device=dev, dtype=torch.float32 if a.f32 else bf)
        ms = timeit(lambda: gemm(A, B, trans_a=a.ta, trans_b=a.tb, out=C, accumulate=a.f32), a.iters, a.warmup, flush)
        tf = 2.0 * a.m * a.n * a.k / ms / 1e9
        out.update(m=a.m, n=a.n, k=a.k, ta=a.ta, tb=a.tb, f32_accumulate=a.f32, ms=ms, tflops=tf,
                   frac_of_peak=tf / tf_peak, peak_source=src)
    elif a.kernel == "gemm_swiglu":
        # gate/up projection with SwiGLU in the epilogue against the plain product followed by the stand-alone kernel
        from . import gemm_swiglu
        X = torch.randn(a.m, a.k, device=dev, dtype=bf)
        W = torch.randn(a.n, a.k, device=dev, dtype=bf) * a.k ** -0.5
        C = torch.empty(a.m, a.n, device=dev, dtype=bf)
        ms = timeit(lambda: gemm_swiglu(X, W), a.iters, a.warmup, flush)
        ms_two = timeit(lambda: swiglu_fwd(gemm(X, W, out=C)), a.iters, a.warmup, flush)
        tf = 2.0 * a.m * a.n * a.k / ms / 1e9
        out.update(m=a.m, n=a.n, k=a.k, ms=ms, tflops=tf, frac_of_peak=tf / tf_peak, gemm_plus_swiglu_kernel_ms=ms_two,
                   peak_source=src)
    elif a.kernel == "gemm_fp8":
        from . import gemm_fp8, quant_blocks_128x128, quant_rows_1x128
        xq, sx = quant_rows_1x128(torch.randn(a.m, a.k, device=dev).to(bf))
        wq, sw = quant_blocks_128x128(torch.randn(a.n, a.k, device=dev).to(bf))
        C = torch.empty(a.m, a.n, device=dev, dtype=bf)
        ms = timeit(lambda: gemm_fp8(xq, sx, wq, sw, out=C), a.iters, a.warmup, flush)
        tf = 2.0 * a.m * a.n * a.k / ms / 1e9
        out.update(m=a.m, n=a.n, k=a.k, ms=ms, tflops=tf, frac_of_bf16_peak=tf / tf_peak, peak_source=src)
    elif a.kernel in ("attn_fwd", "attn_bwd"):
        hd = 128
        qkv = torch.randn(a.batch * a.seq, (a.heads + 2 * a.kv_heads) * hd, device=dev).to(bf)
        o, lse = flash_attn_fwd(qkv, a.batch, a.seq, a.heads, a.kv_heads, hd)
        causal_flops = 4.0 * a.batch * a.heads * a.seq * a.seq * hd / 2
        if a.kernel == "attn_fwd":
            ms = timeit(lambda: flash_attn_fwd(qkv, a.batch, a.seq, a.heads, a.kv_heads, hd, variant=a.variant), a.iters, a.warmup, flush)
            flops = causal_flops
        else:
            do = torch.randn_like(o)
            dqkv = torch.empty_like(qkv)
            delta = torch.empty_like(lse)
            ms = timeit(lambda: flash_attn_bwd(qkv, o, do, lse, a.batch, a.seq, a.heads, a.kv_heads, hd, dqkv=dqkv,
                                               delta=delta, parts=a.parts), a.iters, a.warmup, flush)
            flops = 2.5 * causal_flops
        tf = flops / ms / 1e9
        out.update(batch=a.batch, seq=a.seq, heads=a.heads, kv_heads=a.kv_heads, ms=ms, tflops_useful=tf,
                   frac_of_peak=tf / tf_peak, peak_source=src)
    elif a.kernel == "rmsnorm_bwd":
        x = torch.randn(a.rows, a.hidden, device=dev).to(bf)
        g = torch.ones(a.hidden, device=dev, dtype=bf)
        dy = torch.randn_like(x)
        _, rstd = rmsnorm_fwd(x, g)
        dx = torch.zeros_like(x)
        dg = torch.zeros(a.hidden, device=dev)
        scratch = torch.empty(640 * a.hidden, device=dev)
        ms = timeit(lambda: rmsnorm_bwd(x, g, rstd, dy, dx=dx, dg=dg, dx_accumulate=True, dg_accumulate=True,
                                        scratch=scratch), a.iters, a.warmup, flush)
        gb = 4.0 * a.rows * a.hidden * 2 / 1e9   # x, dy, dx read + dx write
        out.update(rows=a.rows, hidden=a.hidden, ms=ms, gbs=gb / (ms * 1e-3), frac_of_peak=gb / (ms * 1e-3) / bw_peak,
                   peak_source=src)
    else:
        gu = torch.randn(a.rows, 2 * a.ffn, device=dev).to(bf)
        d = torch.randn(a.rows, a.ffn, device=dev).to(bf)
        ms_f = timeit(lambda: swiglu_fwd(gu), a.iters, a.warmup, flush)
        ms_b = timeit(lambda: swiglu_bwd(gu, d), a.iters, a.warmup, flush)
        out.update(rows=a.rows, ffn=a.ffn, fwd_ms=ms_f, bwd_ms=ms_b,
                   fwd_gbs=3.0 * a.rows * a.ffn * 2 / 1e9 / (ms_f * 1e-3),
                   bwd_gbs=5.0 * a.rows * a.ffn * 2 / 1e9 / (ms_b * 1e-3), peak_source=src)
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
