"""Fit the constants of the calibrated pricing backend to a measured op timeline.

    python -m cai_b200.trainer --config my.cfg --steps 5 --trace measured.csv        # on the GPUs
    python -m cai_b200.plan.fit plans/plan.rank000000.bin measured.csv [plan2 trace2 ...] > my_calibration.cfg
    bin/trainer plans/plan.rank000000.bin plans/topology.bin --calibration my_calibration.cfg

Every cost in ``csrc/plan/backend_calibrated.cc`` is linear in its constants once the op's shape is known, so each
group is an ordinary least-squares problem over the ops of that kind in the trace:

  GEMM (per operand class)   t = launch + waves * tile_us + (waves * tile FLOPs) / per-SM rate
  attention                  t = fixed + steps * step_us            (forward; dK / dV and dQ parts of the backward)
  pointwise kernels          t = fixed + operand MB * us_per_mb

Groups with too few distinct shapes in the trace keep their built-in values (they are left out of the output). The
fused tensor-parallel, NCCL and expert-exchange constants describe links, not kernels of one GPU, and are not fitted here.
"""
from __future__ import annotations

import argparse
import math
import sys

import numpy as np

from . import K_GEMM, PlanFile
from .compare import load

SMS = 148
K_RMSNORM_FWD, K_RMSNORM_BWD, K_ROPE, K_ATTN_FWD, K_ATTN_BWD, K_SWIGLU_FWD, K_SWIGLU_BWD = 3, 4, 6, 7, 8, 9, 10
K_CROSS_ENTROPY, K_ADAMW, K_CROSS_ENTROPY_TP, K_EMBED_FWD, K_EMBED_BWD = 11, 12, 29, 1, 2
POINTWISE = {K_RMSNORM_FWD: "rmsnorm_fwd", K_RMSNORM_BWD: "rmsnorm_bwd", K_ROPE: "rope", K_SWIGLU_FWD: "swiglu",
             K_SWIGLU_BWD: "swiglu", K_ADAMW: "adamw", K_CROSS_ENTROPY: "cross_entropy", K_CROSS_ENTROPY_TP: "cross_entropy",
             K_EMBED_FWD: "embed", K_EMBED_BWD: "embed"}


def gemm_features(M, N, K, sms=SMS):
    bn = 256.0 if N % 256 == 0 else 128.0
    tiles = math.ceil(M / 128.0) * math.ceil(N / bn)
    waves = max(1.0, math.ceil(tiles / sms))
    return waves, waves * 2.0 * 128.0 * bn * K


def attention_steps(B, S, nh, nkv, sms=SMS):
    nq = S / 128.0
    tri = nq * (nq + 1.0) / 2.0
    rep = nh / max(1, nkv)
    split = rep > 1 and B * nkv * nq < sms and B * nh * nq <= sms
    return {"fwd": max(B * nh * tri / sms, nq), "dkdv": max(B * nh * tri / sms, (1.0 if split else rep) * nq),
            "dq": max(B * nh * tri / sms, nq)}


def _lstsq(rows, y, names, min_rows):
    """Least squares with non-negative clipping; None when the system is under-determined."""
    A = np.asarray(rows, dtype=np.float64)
    y = np.asarray(y, dtype=np.float64)
    if len(y) < min_rows or np.linalg.matrix_rank(A) < A.shape[1]:
        return None
    sol, *_ = np.linalg.lstsq(A, y, rcond=None)
    pred = A @ sol
    err = float(np.max(np.abs(pred - y) / np.maximum(y, 1e-9)))
    return dict(zip(names, sol)), err


def fit(pairs):
    """``pairs``: ``[(plan file, trace file), ...]`` (several layouts of a model give the fit more distinct shapes).
    Returns ``(constants, report)``: fitted ``key -> value`` pairs and one line per group with its worst relative error."""
    gemm = {0: ([], []), 1: ([], [])}
    attn = {"fwd": ([], []), "dkdv": ([], []), "dq": ([], []), "bwd_all": ([], [])}
    point = {}
    ops = []
    for plan_path, trace_path in pairs:
        pf = PlanFile(plan_path)
        trace = load(trace_path)
        ops += [(pf, op, trace[i][2]) for i, op in enumerate(pf.ops) if op.exec and i in trace]
    for pf, op, us in ops:
        x = pf.exec[op.exec - 1]
        k = int(x.kernel)
        if k == K_GEMM and not (x.flags & 0x100):
            waves, wf = gemm_features(x.i[0], x.i[1], x.i[2])
            rows, ys = gemm[x.flags & 1]
            rows.append([1.0, waves, wf * 1e-6])          # us = launch + waves * tile_us + wf / rate   (rate in FLOP/us)
            ys.append(us)
        elif k in (K_ATTN_FWD, K_ATTN_BWD):
            st = attention_steps(x.i[0], x.i[1], x.i[2], x.i[3])
            if k == K_ATTN_FWD:
                attn["fwd"][0].append([1.0, st["fwd"]]); attn["fwd"][1].append(us)
            else:
                parts = (x.flags & 7) or 7
                if parts == 2:
                    attn["dkdv"][0].append([1.0, st["dkdv"]]); attn["dkdv"][1].append(us)
                elif parts == 4:
                    attn["dq"][0].append([1.0, st["dq"]]); attn["dq"][1].append(us)
                elif parts == 7:
                    attn["bwd_all"][0].append([1.0, st["dkdv"], st["dq"]]); attn["bwd_all"][1].append(us)
        elif k in POINTWISE:
            mb = sum(pf.tensors[t].nbytes for t in x.t if 0 <= t < len(pf.tensors)) / 1e6
            rows, ys = point.setdefault(POINTWISE[k], ([], []))
            rows.append([1.0, mb]); ys.append(us)
    out, report = {}, []

    def take(label, res, mapping):
        if res is None:
            report.append(f"# {label}: not enough distinct shapes in the trace, built-in values kept")
            return
        sol, err = res
        for key, fn in mapping.items():
            v = fn(sol)
            if v is not None and np.isfinite(v) and v > 0:
                out[key] = float(v)
        report.append(f"# {label}: worst relative error of the fit {err * 100:.1f} %")

    for cls, suffix in ((0, ""), (1, "_ta")):
        rows, ys = gemm[cls]
        res = _lstsq(rows, ys, ("launch", "tile", "inv_rate"), 4)
        take("GEMM, A transposed" if cls else "GEMM", res,
             {"gemm_tile_us" + suffix: lambda s: max(s["tile"], 0.0) or None,
              "gemm_sm_flops" + suffix: lambda s: 1e12 / s["inv_rate"] if s["inv_rate"] > 0 else None,
              **({"gemm_launch_us": lambda s: max(s["launch"], 0.0) or None} if cls == 0 else {})})
    take("attention forward", _lstsq(*attn["fwd"], ("fixed", "step"), 2),
         {"attn_fwd_fixed_us": lambda s: s["fixed"], "attn_fwd_step_us": lambda s: s["step"]})
    if attn["dkdv"][1] or attn["dq"][1]:     # tensor-parallel plans launch the parts separately (both carry the fixed cost)
        take("attention backward, dK / dV", _lstsq(*attn["dkdv"], ("fixed", "step"), 2),
             {"attn_bwd_fixed_us": lambda s: s["fixed"], "attn_dkdv_step_us": lambda s: s["step"]})
        take("attention backward, dQ", _lstsq(*attn["dq"], ("fixed", "step"), 2), {"attn_dq_step_us": lambda s: s["step"]})
    else:
        take("attention backward (whole)", _lstsq(*attn["bwd_all"], ("fixed", "dkdv", "dq"), 3),
             {"attn_bwd_fixed_us": lambda s: s["fixed"], "attn_dkdv_step_us": lambda s: s["dkdv"], "attn_dq_step_us": lambda s: s["dq"]})
    for name, (rows, ys) in sorted(point.items()):
        take(name, _lstsq(rows, ys, ("fixed", "slope"), 2),
             {f"{name}_fixed_us": lambda s: s["fixed"], f"{name}_us_per_mb": lambda s: s["slope"]})
    return out, report


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("files", nargs="+", help="plan file and the measured op timeline of that rank (CSV or Trace Event JSON), "
                    "repeated for every layout measured: plan1 trace1 [plan2 trace2 ...]")
    a = ap.parse_args(argv)
    if len(a.files) % 2:
        ap.error("plan and trace files come in pairs")
    pairs = list(zip(a.files[0::2], a.files[1::2]))
    consts, report = fit(pairs)
    print(f"# calibration fitted from {', '.join(t for _, t in pairs)}; constants not listed keep their built-in values")
    for line in report:
        print(line)
    for k in sorted(consts):
        print(f"{k} = {consts[k]:.6g}")
    return 0 if consts else 1


if __name__ == "__main__":
    sys.exit(main())
