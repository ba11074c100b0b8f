"""Rank the parallel layouts of a model on a given number of GPUs without touching a GPU.

For every layout the executable-plan compiler accepts (tensor x pipeline x data / expert parallel, optimizer-state or
full ZeRO-3 sharding), the plans of one rank per pipeline stage are compiled and replayed by the calibrated pricing
backend (costs fitted to this repository's kernels as measured on B200s; the stages of a pipeline are replayed together,
their sends meeting their receives); the table gives the predicted step time,
tokens/s and the arena a rank allocates. The global batch of the input configuration is kept (``grad_accum`` follows the
data-parallel degree). This is the offline question the reference's simulator is for ("which decomposition?",
tools/topology_linter.c suggests tensor-parallel sizes by rule); here the answer comes from measured kernel costs.

    python -m cai_b200.plan.advise configs/b200_tp8.cfg --gpus 8
"""
from __future__ import annotations

import argparse
import os
import tempfile
from pathlib import Path

from . import PlanError, PlanFile, Simulator, compile_plans, describe, pipeline_replay, set_log_level


def _divisors(n, limit):
    return [d for d in range(1, min(n, limit) + 1) if n % d == 0]


def candidates(base: dict, world: int, mb_groups=(0,)):
    """Layouts worth pricing: tp divides the kv heads (<= 8, one NVLink domain), pp divides the layers, the rest is data
    (and, for MoE, expert) parallel; ZeRO-3 where the compiler has an executable schedule for it. ``mb_groups``:
    microbatches per launch to try (0 = the compiler's choice)."""
    global_batch = base["global_batch"]
    for tp in _divisors(base["num_kv_heads"], 8):
        for pp in _divisors(base["num_layers"], 8):
            if world % (tp * pp):
                continue
            dp = world // (tp * pp)
            per_replica = base["microbatch"] * dp
            if global_batch % per_replica:
                continue
            grad_accum = global_batch // per_replica
            if pp > 1 and grad_accum < pp:
                continue
            stages = (1,) if dp == 1 or base["is_moe"] else (1, 2, 3) if tp == 1 else (1, 3)      # ZeRO-2 shards gradients through the tp = 1 buckets
            for zero in stages:
                for g in mb_groups:
                    if g and (grad_accum % g or pp > 1 or zero == 3 or base["is_moe"]):
                        continue        # grouping exists for dense, unpipelined, ZeRO-1 schedules only
                    yield {"tp": tp, "pp": pp, "dp": dp, "ep": dp if base["is_moe"] else 1, "zero_stage": zero,
                           "grad_accum": grad_accum, "mb_group": g}


def evaluate(config_text: str, cand: dict, world: int, backend: str = "calibrated", workdir=None, calibration=None) -> dict:
    text = (config_text + f"\ngpus_per_rack = {world}\ntrays_per_rack = 1\ngpus_per_tray = {world}\nnum_racks = 1\n"
            f"tp = {cand['tp']}\npp = {cand['pp']}\nep = {cand['ep']}\nzero_stage = {cand['zero_stage']}\n"
            f"grad_accum = {cand['grad_accum']}\ncomm = fused\nmb_group = {cand.get('mb_group', 0)}\n")
    out = dict(cand)
    with tempfile.TemporaryDirectory(dir=workdir) as tmp:
        try:
            compile_plans(text, tmp, ranks=(0, world), version=2, text=True)
        except PlanError as e:
            out["note"] = str(e).split("): ", 1)[-1][:90]
            return out
        stage_rank = {}
        for r in range(world):
            pf = PlanFile(Path(tmp) / f"plan.rank{r:06d}.bin")
            stage_rank.setdefault(pf.hdr.pipeline_stage, (r, pf.hdr.arena_bytes))
        if cand["pp"] > 1:
            # all stages replayed together: sends meet their receives, no closed bubble formula
            paths = [Path(tmp) / f"plan.rank{stage_rank[s][0]:06d}.bin" for s in sorted(stage_rank)]
            step = pipeline_replay(paths, Path(tmp) / "topology.bin", backend=backend, calibration=calibration)["step_time_s"]
        else:
            r = stage_rank[0][0]
            sim = Simulator(Path(tmp) / f"plan.rank{r:06d}.bin", Path(tmp) / "topology.bin", rank=r, backend=backend,
                            calibration=calibration)
            step = sim.step().step_time_s
            sim.close()
        d = describe(text)
        out.update(step_ms=step * 1e3, tokens_per_s=d["global_tokens"] / step,
                   arena_gib=max(a for _, a in stage_rank.values()) / 2**30,
                   fits=max(a for _, a in stage_rank.values()) <= d["mem_budget"])
    return out


def advise(config_path, gpus=None, backend="calibrated", mb_groups=(0,), calibration=None):
    text = Path(config_path).read_text()
    base = describe(text)
    world = gpus or base["world_size"]
    rows = [evaluate(text, c, world, backend, calibration=calibration) for c in candidates(base, world, mb_groups)]
    ok = sorted((r for r in rows if "step_ms" in r), key=lambda r: (not r["fits"], r["step_ms"]))
    return ok, [r for r in rows if "step_ms" not in r]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("config")
    ap.add_argument("--gpus", type=int, default=None, help="GPUs of one NVLink domain (default: the configuration's)")
    ap.add_argument("--backend", default="calibrated", choices=("calibrated", "analytic"))
    ap.add_argument("--top", type=int, default=12)
    ap.add_argument("--mb-groups", default="0", help="microbatches per launch to try, comma separated (0 = the compiler's choice)")
    ap.add_argument("--calibration", help="key = value file overriding constants of the calibrated backend (see configs/b200_calibration.cfg)")
    a = ap.parse_args(argv)
    if "CAI_LOG_LEVEL" not in os.environ:
        set_log_level("warn")       # one table on stdout; the per-plan INFO lines of dozens of replays are noise here
    ok, refused = advise(a.config, a.gpus, a.backend, tuple(int(x) for x in a.mb_groups.split(",")), a.calibration)
    print(f"{'tp':>3} {'pp':>3} {'dp':>3} {'ep':>3} {'zero':>4} {'accum':>5} {'group':>5} | {'step ms':>9} | {'tokens/s':>10} | {'arena GiB':>9} | fits")
    for r in ok[:a.top]:
        print(f"{r['tp']:3d} {r['pp']:3d} {r['dp']:3d} {r['ep']:3d} {r['zero_stage']:4d} {r['grad_accum']:5d} {r['mb_group']:5d} | {r['step_ms']:9.1f} | "
              f"{r['tokens_per_s']:10.3e} | {r['arena_gib']:9.2f} | {'yes' if r['fits'] else 'NO'}")
    for r in refused:
        print(f"{r['tp']:3d} {r['pp']:3d} {r['dp']:3d} {r['ep']:3d} {r['zero_stage']:4d} {r['grad_accum']:5d} {r['mb_group']:5d} | not executable: {r['note']}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
