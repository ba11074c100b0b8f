"""Continue a run after GPUs were lost and no spare is left: pick the best layout for the GPUs that remain and
rearrange the last checkpoint for it.

    python -m cai_b200.utils.elastic --config run.cfg --lost 1 --ckpt ckpt/run --out-config run_shrunk.cfg --out-ckpt ckpt/run_shrunk
    ./launch.sh plans_shrunk/ python -m cai_b200.trainer --ckpt ckpt/run_shrunk ...

With spares (``spare_gpus`` in the configuration) a failed rank is replaced one for one and nothing else changes: that
is ``bin/plan_recover`` (the reference's tools/plan_recover.c), and this tool says so. Without spares the reference
stops (elastic recovery is on its roadmap only); here the job shrinks. Every executable layout on the remaining GPUs -
and on fewer, when the remaining count divides badly (7 GPUs rarely tile a model) - is priced with the calibrated
backend (pipelined layouts with all stages replayed together), the global batch is kept (``grad_accum`` absorbs the
smaller data-parallel degree) so the optimisation follows the same trajectory, the fastest layout that fits in memory
is written as a configuration, and the rolling "latest" checkpoint is re-sharded for it. Host only; no GPU is touched.
"""
from __future__ import annotations

import argparse
import os
from pathlib import Path

from ..plan import describe, set_log_level
from ..plan.advise import candidates, evaluate
from . import reshard as resharder


def layout_keys(cand: dict, world: int) -> str:
    """The configuration lines that place ``cand`` on ``world`` GPUs of one NVLink domain (later keys override earlier)."""
    return (f"\n# layout chosen by cai_b200.utils.elastic for {world} GPUs\n"
            f"gpus_per_rack = {world}\ntrays_per_rack = 1\ngpus_per_tray = {world}\nnum_racks = 1\nspare_gpus = 0\n"
            f"tp = {cand['tp']}\npp = {cand['pp']}\nep = {cand['ep']}\nzero_stage = {cand['zero_stage']}\n"
            f"grad_accum = {cand['grad_accum']}\nmb_group = {cand.get('mb_group', 0)}\n")


def shrink(config_text: str, gpus_left: int, backend: str = "calibrated", calibration=None):
    """Best layout on at most ``gpus_left`` GPUs. Returns ``(world, layout row)`` or ``(0, None)`` when nothing executable
    fits. Rows are those of ``cai_b200.plan.advise``; a layout on fewer GPUs wins only by predicted throughput."""
    base = describe(config_text)
    best_world, best = 0, None
    for world in range(gpus_left, 0, -1):
        for cand in candidates(base, world):
            row = evaluate(config_text, cand, world, backend, calibration=calibration)
            if "step_ms" not in row or not row["fits"]:
                continue
            if best is None or row["step_ms"] < best["step_ms"]:
                best_world, best = world, row
    return best_world, best


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", required=True, help="configuration of the run that lost GPUs")
    g = ap.add_mutually_exclusive_group(required=True)
    g.add_argument("--lost", type=int, help="number of GPUs that are gone")
    g.add_argument("--gpus-left", type=int, help="number of GPUs that remain")
    ap.add_argument("--ckpt", help="checkpoint path prefix of the run (as given to the trainer's --ckpt)")
    ap.add_argument("--out-config", required=True, help="where to write the configuration of the shrunk run")
    ap.add_argument("--out-ckpt", help="checkpoint path prefix to write for the new layout (needed with --ckpt)")
    ap.add_argument("--backend", default="calibrated", choices=("calibrated", "analytic"))
    ap.add_argument("--calibration", help="key = value file overriding constants of the calibrated backend")
    a = ap.parse_args(argv)
    if a.ckpt and not a.out_ckpt:
        ap.error("--ckpt needs --out-ckpt")
    if "CAI_LOG_LEVEL" not in os.environ:
        set_log_level("warn")
    text = Path(a.config).read_text()
    base = describe(text)
    world = base["world_size"]
    left = a.gpus_left if a.gpus_left is not None else world - a.lost
    if left < 1 or left >= world:
        print(f"nothing to do: the run has {world} GPUs, {left} would remain")
        return 2
    spares = base.get("spare_gpus", 0)
    if spares >= world - left:
        print(f"the configuration keeps {spares} spare GPU(s): substitute the failed rank(s) with bin/plan_recover "
              f"{a.config} <failed_rank> <outdir> and restore that rank's latest checkpoint; the layout does not change")
        return 0
    new_world, best = shrink(text, left, a.backend, a.calibration)
    if best is None:
        print(f"no executable layout of this model fits on {left} or fewer GPUs")
        return 1
    Path(a.out_config).write_text(text + layout_keys(best, new_world))
    print(f"{world} -> {left} GPUs: tp {best['tp']} x pp {best['pp']} x dp {best['dp']}"
          + (f" (ep {best['ep']})" if best["ep"] > 1 else "") + (", ZeRO-3" if best["zero_stage"] == 3 else "")
          + f" on {new_world} GPUs, grad_accum {best['grad_accum']} (global batch kept), predicted {best['step_ms']:.1f} ms/step, "
          f"{best['tokens_per_s']:.3e} tokens/s, arena {best['arena_gib']:.2f} GiB")
    if new_world < left:
        print(f"({left - new_world} of the remaining GPUs stay idle: no layout on {left} divides the model and the batch, or none is faster)")
    print(f"wrote {a.out_config}")
    if a.ckpt:
        step, n, ranks = resharder.reshard(a.config, a.ckpt, a.out_config, a.out_ckpt)
        print(f"step {step}: {n} parameters (master, m, v) rearranged for {ranks} ranks -> {a.out_ckpt}.latest.rank*")
    print(f"next: bin/plan_compiler {a.out_config} <plans> --exec --all && ./launch.sh <plans> python -m cai_b200.trainer"
          + (f" --ckpt {a.out_ckpt}" if a.ckpt else ""))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
