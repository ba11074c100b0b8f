#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s, MFU) of the dense 24-layer / hidden-2048
decoder of ``configs/b200_tp8.cfg`` on N GPUs of one B200 box, tensor parallel over the N GPUs
(tp = N, the named config at N = 8). Global batch is fixed (grad_accum 8 x seq 4096), so scaling
over N is strong scaling.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torch.distributed.run)

Two measurements per run, both over EXACTLY K optimizer steps after W warm-up steps:
  * ``value``: device-timed (CUDA events on the launching stream, barrier + synchronize on both
    sides, max over ranks) with the batch already resident on the device;
  * ``e2e``: the same steps through the public API ``Engine.step`` - every step copies its
    tokens/targets from pinned host memory to the device and reads the loss back.
The working set (3 GB of bf16 weights, >7 GB of activations per microbatch) is far larger than the
126 MB L2, so no explicit L2 flush is needed between iterations.

``--impl reference`` runs the unmodified reference, built by its own Makefile into ``baseline/_ref``
(``cai_b200/_build.py:build_reference``), through its stock GPU entry point ``gpu_trainer``. That
executable can only train its hard-coded 88k-parameter model, so its line carries
``same_config: false``; both arms also print ``useful_flops_per_s`` (6 x parameters x tokens/s, plus the
attention term for this framework's arm) so that the work rates can be compared across the two models.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SIM_BASELINE_TOKENS_PER_S_TP8 = 7.55e5  # reference simulator's prediction for this config at tp=8


# The named configs of the benchmark set and how each spreads over N GPUs of one box.
CONFIGS = {
    "tp8": ("b200_tp8.cfg", "dense 24L h2048 ffn8192 16h/8kv hd128 V32000 (configs/b200_tp8.cfg)", "tp"),
    "fsdp8b": ("b200_fsdp8b.cfg", "dense 8B 32L h4096 ffn14336 32h/8kv V128256 seq8192, ZeRO-3 + fp8 linear layers "
               "(configs/b200_fsdp8b.cfg)", "dp"),
    "moe_ep8": ("b200_moe_ep8.cfg", "MoE 16L h4096 64 experts ffn1536 top-8 (configs/b200_moe_ep8.cfg)", "ep"),
    "pp2tp4": ("b200_pp2tp4.cfg", "dense 48L h6144 ffn24576 48h/8kv, 1F1B, full recompute (configs/b200_pp2tp4.cfg)", "pp2"),
}


def config_text(n_gpus: int, comm: str, name: str = "tp8", extra: str = "") -> str:
    fname, _, how = CONFIGS[name]
    base = (ROOT / "configs" / fname).read_text()
    text = base + f"\ngpus_per_rack = {n_gpus}\ntrays_per_rack = 1\ngpus_per_tray = {n_gpus}\ncomm = {comm}\n" + extra
    if how == "tp":
        text += f"tp = {n_gpus}\n"
    elif how == "ep":
        text += f"ep = {n_gpus}\n"          # data parallel over all GPUs, experts sharded over the same group
    elif how == "pp2":
        text += f"pp = {2 if n_gpus > 1 else 1}\ntp = {max(1, n_gpus // 2)}\n"
    return text


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, path):
        self.path, self.proc = path, None

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, gpu_index=0):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        clocks, reasons, smax = [], set(), None
        for line in Path(self.path).read_text().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9 or not c[0].isdigit() or int(c[0]) != gpu_index:
                continue
            try:
                clocks.append(float(c[1]))
                smax = float(c[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if clocks:
            busy = sorted(clocks)[len(clocks) // 4:]  # drop the idle tail of the sampling window
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=smax, reasons=sorted(reasons), samples=len(clocks))
        return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from cai_b200.runtime.engine import Engine, synthetic_batch

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    extra = "".join(f"{kv.replace('=', ' = ')}\n" for kv in args.set)
    eng = Engine(config_text=config_text(world, args.comm, args.config, extra), rank=rank, world=world, local_rank=local)
    m = eng.model
    rows = eng.hdr.num_microbatches * m.microbatch
    K, W = args.steps, max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    dp_id = rank // max(1, int(eng.hdr.tp) * int(eng.hdr.num_stages))   # every data-parallel replica draws its own rows
    batches = [synthetic_batch(m.vocab_size, m.seq_len, rows, step=s, seed=7, rank_offset=dp_id) for s in range(2)]
    loss0 = None
    for s in range(W):
        l = eng.step(*batches[s % 2])
        loss0 = l if loss0 is None else loss0
    if args.graph:
        eng.use_graph(True)
        eng.step(*batches[0])  # capture + first replay

    sampler = ClockSampler(os.path.join(tempfile.gettempdir(), f"cai_bench_clocks_n{world}_{os.getpid()}.csv")) if rank == 0 else None
    if sampler:
        sampler.start()

    # ---- device-timed: batch resident on the device
    eng.load_batch(*batches[0])
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(eng.stream):
        start.record()
    for _ in range(K):
        eng.run_step()
    with torch.cuda.stream(eng.stream):
        stop.record()
    barrier()
    dev_ms = start.elapsed_time(stop) / K
    launches = eng.launches_per_step * K
    loss_dev = eng.read_loss()

    # ---- end to end through Engine.step: H2D of inputs and D2H of the loss every step
    barrier()
    t0 = time.perf_counter()
    h2d = 0
    for s in range(K):
        tok, tgt = batches[s % 2]
        h2d = eng.load_batch(tok, tgt)
        eng.run_step()
        loss_e2e = eng.read_loss()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / K
    clocks = sampler.stop(gpu_index=local) if sampler else None

    if args.breakdown:
        # per-op CUDA events over one more step, summed per kernel and GEMM shape (rank 0 prints the table)
        import collections
        from cai_b200 import plan as planlib
        recs = eng.trace_step(*batches[0])
        agg = collections.defaultdict(lambda: [0.0, 0, 0.0])
        for r in recs:
            op = eng.plan.ops[r.op_index]
            x = eng.plan.exec[op.exec - 1]
            key = planlib.KERNEL_NAMES[x.kernel]
            if x.kernel in (planlib.K_GEMM, 20, 21, planlib.K_GEMM_FP8):
                key += f"_ta{x.flags & 1}tb{(x.flags >> 1) & 1}_M{x.i[0]}N{x.i[1]}K{x.i[2]}"
            a = agg[key]
            a[0] += r.end_s - r.start_s
            a[1] += 1
            a[2] += op.flops
        if rank == 0:
            tot = sum(a[0] for a in agg.values())
            print(f"# per-op breakdown of one step, {world} GPU(s), {tot * 1e3:.1f} ms traced", file=sys.stderr)
            for k, a in sorted(agg.items(), key=lambda kv: -kv[1][0])[:30]:
                print(f"# {k:48s} {a[0] * 1e3:9.2f} ms {100 * a[0] / tot:5.1f}% n={a[1]:5d} {a[2] / max(a[0], 1e-9) / 1e12:8.1f} TFLOP/s",
                      file=sys.stderr)

    t = torch.tensor([dev_ms, e2e_ms], device=eng.device, dtype=torch.float64)
    # the loss lives on the last pipeline stage (the other stages read 0): every rank reports the largest value
    lv = torch.tensor([loss0 or 0.0, loss_e2e, loss_dev], device=eng.device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(lv, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()
    loss0, loss_e2e, loss_dev = lv.tolist()
    tokens = eng.tokens_per_step()
    value = tokens / (dev_ms * 1e-3)
    peaks = {}
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    measured_peak = peaks.get("bf16_tflops_sustained", 1400.0) * 1e12
    if rank == 0:
        line = {
            "metric": "tokens/s (whole job), device-timed training step",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / SIM_BASELINE_TOKENS_PER_S_TP8) if (world == 8 and args.config == "tp8") else None,
            "baseline_note": "reference publishes no measured number; ratio is against its analytic simulator's "
                             "prediction for tp=8 (7.55e5 tokens/s), given only at N=8",
            "dtype": "bf16" if m.param_dtype != 3 else "fp8e4m3 linear layers, bf16 elsewhere", "data": "synthetic uniform-random tokens, random-init N(0,0.02) weights",
            "impl": "cai_b200",
            "config": {"model": CONFIGS[args.config][1],
                       "global_batch": int(eng.hdr.grad_accum * m.microbatch * eng.hdr.dp), "seq_len": int(m.seq_len),
                       "parallelism": f"tp{eng.hdr.tp} pp{eng.hdr.num_stages} dp{eng.hdr.dp} ep{eng.hdr.ep}", "microbatch": int(m.microbatch), "grad_accum": int(eng.hdr.grad_accum),
                       "comm": args.comm, "cuda_graph": bool(args.graph),
                       "microbatches_per_launch": int(eng.batch_cols // (m.microbatch * m.seq_len)), "overrides": list(args.set),
                       "l2": "working set (>10 GB per step) exceeds the 126 MB L2; no explicit flush"},
            "useful_flops_per_s": float(eng.hdr.flops_per_token_useful) * value,
            "mfu_vs_2.25PF": eng.mfu(dev_ms * 1e-3, 2.25e15),
            "mfu_vs_measured_sustained": eng.mfu(dev_ms * 1e-3, measured_peak),
            "loss_first": loss0, "loss_last": loss_e2e, "loss_after_device_timed": loss_dev,
            "clocks": clocks,
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 32},
            "gpu_launches": int(launches),
        }
        print(json.dumps(line), flush=True)
    eng.close()
    if world > 1 and dist.is_initialized():
        dist.destroy_process_group()


REF_SPEC = {"vocab": 64, "seq": 32, "hidden": 64, "layers": 2, "heads": 4, "head_dim": 16, "ffn": 128, "batch_per_rank": 16}
REF_ID_FILES = ("/tmp/cai_nccl_dp_0.id",)   # the reference's NCCL bootstrap file for pure data parallel; it never deletes it


def _run_gpu_trainer(exe, steps, timeout_s):
    """Run the reference's gpu_trainer (its stock main) with stdout on a pseudo-terminal, so that its per-step
    `step N  loss X` lines arrive when they are printed (each follows the step's device->host loss read), and
    return [(step, seconds since launch, loss)], the exit code and the tail of its stderr."""
    import pty
    import re
    import select
    master, slave = pty.openpty()
    t0 = time.perf_counter()
    proc = subprocess.Popen([str(exe), "--steps", str(steps), "--batch", str(REF_SPEC["batch_per_rank"])],
                            stdout=slave, stderr=subprocess.PIPE, stdin=subprocess.DEVNULL)
    os.close(slave)
    pat = re.compile(rb"step\s+(\d+)\s+loss\s+(\S+)")
    lines, buf = [], b""
    deadline = t0 + timeout_s
    while True:
        if time.perf_counter() > deadline:
            proc.kill()          # our own child, by handle
            break
        r, _, _ = select.select([master], [], [], 0.2)
        if r:
            try:
                chunk = os.read(master, 65536)
            except OSError:
                chunk = b""
            now = time.perf_counter() - t0
            if not chunk:
                break
            buf += chunk
            while b"\n" in buf:
                line, buf = buf.split(b"\n", 1)
                m = pat.search(line)
                if m:
                    try:
                        lines.append((int(m.group(1)), now, float(m.group(2))))
                    except ValueError:
                        lines.append((int(m.group(1)), now, float("nan")))
        elif proc.poll() is not None:
            break
    rc = proc.wait()
    err = proc.stderr.read().decode(errors="replace")[-400:] if proc.stderr else ""
    os.close(master)
    return lines, rc, err


def run_reference(args):
    """The reference arm: the UNMODIFIED reference, built by its own Makefile (`make CUDA=1 NCCL=1`, see
    cai_b200/_build.py:build_reference), run through its stock GPU entry point tools/gpu_trainer.c. That
    executable trains a hard-coded 88k-parameter model (vocab 64, seq 32, hidden 64, 2 layers, MHA 4 x 16, ffn
    128) in pure data parallel with naive fp32 kernels; it has no way to run the headline model (no GQA, RoPE,
    tensor-parallel split or vocabulary of 32000: tools/gpu_trainer.c:38-46), so the line says
    `same_config: false`. Its step already copies the batch host->device and the per-row losses device->host
    (src/cuda/cai_gpu_train.cu:273-293), so the one measurement is end to end."""
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))

    def say(obj):
        if rank == 0:
            obj = {"impl": "reference", **obj}
            print(json.dumps(obj), flush=True)

    exe = ROOT / "baseline" / "_ref" / "bin" / "gpu_trainer"
    if not exe.exists() and rank == 0:
        try:
            from cai_b200 import _build
            _build.build_reference()
        except Exception:
            pass
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group(backend="gloo", rank=rank, world_size=world)   # host-side barrier of this harness only
        dist.barrier()
    if not exe.exists():
        log = ROOT / "baseline" / "_ref" / "BUILD_LOG.txt"
        why = log.read_text().strip().splitlines()[-1][:160] if log.exists() else "no build log"
        say({"unavailable": f"reference gpu_trainer could not be built here (make CUDA=1 NCCL=1): {why}"})
        return
    K, W = args.steps, max(args.warmup, 3)
    if rank == 0:
        for f in REF_ID_FILES:      # a stale id file makes the other ranks join a communicator that no longer exists
            try:
                os.unlink(f)
            except OSError:
                pass
    if dist:
        dist.barrier()
    sampler = ClockSampler(os.path.join(tempfile.gettempdir(), f"cai_ref_clocks_n{world}_{os.getpid()}.csv")) if rank == 0 else None
    if sampler:
        sampler.start()
    lines, rc, err = _run_gpu_trainer(exe, W + K, timeout_s=180)   # a run takes seconds; a hung NCCL bootstrap must not hold the job
    clocks = sampler.stop(gpu_index=int(os.environ.get("LOCAL_RANK", 0))) if sampler else None
    ok = rc == 0 and len(lines) >= 2
    # steps are printed every max(1, (W+K)//20) steps: the timed span starts at the first line at or past the
    # warm-up and ends at the last one
    span = [l for l in lines if l[0] >= W - 1]
    if ok and len(span) >= 2:
        n_steps = span[-1][0] - span[0][0]
        ms = (span[-1][1] - span[0][1]) * 1e3 / n_steps
    else:
        ok, n_steps, ms = False, 0, 0.0
    if dist:
        import torch
        t = torch.tensor([ms if ok else -1.0], dtype=torch.float64)
        lo = t.clone()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        if rank == 0:       # only rank 0 of the reference prints steps; the others report -1 and are ignored
            ms = float(t.item())
        dist.barrier()
        if rank == 0:
            for f in REF_ID_FILES:
                try:
                    os.unlink(f)
                except OSError:
                    pass
        dist.destroy_process_group()
    if not ok:
        say({"unavailable": f"reference gpu_trainer exited {rc} after {len(lines)} step lines: {err.strip()[-200:]}"})
        return
    bt = REF_SPEC["batch_per_rank"] * REF_SPEC["seq"]
    tokens = bt * world
    value = tokens / (ms * 1e-3)
    say({
        "metric": "tokens/s (whole job), training step of the reference's gpu_trainer, timed from its own step lines",
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "steps_timed": n_steps,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic (the reference's own xorshift token stream), its own random init",
        "same_config": False,
        "useful_flops_per_s": 6.0 * 88384 * value,
        "config": {"model": "reference's hard-coded model: 2L h64 4x16 heads ffn128 V64 seq32 (88,384 parameters); it cannot "
                            "run the headline model", "global_batch": REF_SPEC["batch_per_rank"] * world,
                   "seq_len": REF_SPEC["seq"], "parallelism": f"dp{world}",
                   "timing": "wall clock between the executable's step lines (each printed after the step's loss reached the host)"},
        "loss_first": lines[0][2], "loss_last": lines[-1][2],
        "clocks": clocks,
        "e2e": {"value": value, "unit": "tokens/s", "ms_per_step": ms, "h2d_bytes_per_step": 2 * bt * 4, "d2h_bytes_per_step": bt * 4},
    })


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--comm", default="fused", choices=["fused", "baseline"])
    ap.add_argument("--graph", type=int, default=0)
    ap.add_argument("--breakdown", action="store_true", help="also print a per-op time table of one step (stderr)")
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE",
                    help="override a key of the config file (schedule options such as mb_group=1); repeatable")
    ap.add_argument("--config", default="tp8", choices=sorted(CONFIGS), help="which named config (default: the headline one)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
