"""Device trainer: one process == one GPU rank.

    python -m cai_b200.trainer <plan.bin> <topology.bin> [--steps N] [--ckpt PATH] [--ckpt-every K]
                               [--trace CSV] [--graph] [--nvtx] [--jsonl FILE]
    python -m cai_b200.trainer --config configs/x.cfg [...]        (compiles this rank's plan first)

Same command line, table and checkpoint naming as the reference's ``trainer`` (tools/trainer.c),
but the plan is executed on the GPU: real kernels, measured step time / MFU / tokens/s, a loss
column, measured per-stream occupancy, an op timeline with measured times, and checkpoints that
carry parameters and optimizer state. Rank and world size come from RANK / WORLD_SIZE / LOCAL_RANK
(``tools/launch.sh`` or ``torch.distributed.run`` set them). Data is a synthetic uniform-random
token stream, a different slice per data-parallel replica.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

from . import plan as planlib
from .runtime.engine import Engine, synthetic_batch


def main(argv=None):
    ap = argparse.ArgumentParser(prog="cai_b200.trainer")
    ap.add_argument("plan", nargs="?")
    ap.add_argument("topology", nargs="?")
    ap.add_argument("--config")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--ckpt")
    ap.add_argument("--ckpt-every", type=int, default=0)
    ap.add_argument("--trace")
    ap.add_argument("--graph", action="store_true")
    ap.add_argument("--nvtx", action="store_true", help="NVTX range per op, named by kernel (for timeline tools)")
    ap.add_argument("--jsonl")
    ap.add_argument("--comm", choices=["fused", "baseline"])
    a = ap.parse_args(argv)
    if not a.config and not (a.plan and a.topology):
        ap.print_usage(sys.stderr)
        return 2
    rank = int(os.environ.get("RANK", 0))
    try:
        if a.config:
            eng = Engine(a.config, comm=a.comm)
        else:
            cfg_text = None
            side = os.path.join(os.path.dirname(a.plan), "config.cfg")
            if os.path.exists(side):
                cfg_text = open(side).read()
            eng = Engine(plan_path=a.plan, topology_path=a.topology, config_text=cfg_text)
    except planlib.PlanError as e:
        print(f"init failed: {e}", file=sys.stderr)
        return 1
    ckpt_every = a.ckpt_every or (5 if a.ckpt else 0)
    if a.ckpt:
        try:
            if eng.load_checkpoint(a.ckpt):
                print(f"[cai INFO] resumed from checkpoint at step {eng.step_count}", file=sys.stderr)
        except planlib.PlanError as e:
            print(f"checkpoint rejected: {e}", file=sys.stderr)
            return 1
    m, h = eng.model, eng.hdr
    rows = h.num_microbatches * m.microbatch
    replica = h.tp * h.num_stages * h.cp
    dp_id = rank // replica
    is_printer = rank == (h.num_stages - 1) * h.tp * h.cp  # first rank of the last stage sees the loss
    if is_printer:
        print("step | step_time | bubble |   MFU  | tokens/s    | tok/s/gpu |   loss")
        print("-----+-----------+--------+--------+-------------+-----------+--------")
    sink = open(a.jsonl, "a") if (a.jsonl and is_printer) else None
    bubble = (h.num_stages - 1) / (h.num_microbatches + h.num_stages - 1) if h.num_stages > 1 else 0.0
    sum_mfu = sum_tps = 0.0
    n = 0
    start_ev, stop_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first = eng.step_count
    if a.nvtx:
        eng.nvtx(True)
    try:
        for step in range(first, a.steps):
            tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows * h.dp, step=step, seed=eng.train.seed)
            tok = tok[dp_id * rows:(dp_id + 1) * rows].contiguous().pin_memory()
            tgt = tgt[dp_id * rows:(dp_id + 1) * rows].contiguous().pin_memory()
            if a.graph and step == first + 1:
                eng.use_graph(True)
            if a.trace and step == a.steps - 1:
                recs = eng.trace_step(tok, tgt)
                with open(a.trace, "w") as f:
                    f.write("op_index,kind,stream,start_us,end_us,dur_us,bytes,flops\n")
                    for r in recs:
                        f.write(f"{r.op_index},{planlib.OP_NAMES[r.kind]},{planlib.STREAMS[r.stream]},{r.start_s * 1e6:.4f},"
                                f"{r.end_s * 1e6:.4f},{(r.end_s - r.start_s) * 1e6:.4f},{r.bytes},{r.flops}\n")
                if is_printer:
                    print(f"wrote op timeline to {a.trace}")
                continue
            eng.load_batch(tok, tgt)
            with torch.cuda.stream(eng.stream):
                start_ev.record()
            eng.run_step()
            with torch.cuda.stream(eng.stream):
                stop_ev.record()
            loss = eng.read_loss()
            dt = start_ev.elapsed_time(stop_ev) * 1e-3
            tps = h.global_tokens_per_step / dt
            mfu = eng.mfu(dt)
            if is_printer:
                print(f"{step:4d} | {dt * 1e3:7.2f} ms| {bubble * 100:5.1f}% | {mfu * 100:5.1f}% | {tps:9.2e} | "
                      f"{tps / h.world_size:9.1f} | {loss:7.4f}", flush=True)
                if sink:
                    sink.write(json.dumps({"step": step, "step_time_s": dt, "mfu": mfu, "tokens_per_s": tps,
                                           "loss": loss, "time": time.time()}) + "\n")
                    sink.flush()
            sum_mfu += mfu
            sum_tps += tps
            n += 1
            if ckpt_every and a.ckpt and eng.step_count % ckpt_every == 0:
                eng.save_checkpoint(a.ckpt, "periodic")
    except Exception as e:  # a failed step leaves an emergency checkpoint behind, like the reference
        print(f"step {eng.step_count} failed: {e}", file=sys.stderr)
        if a.ckpt:
            try:
                eng.save_checkpoint(a.ckpt, "emergency", wait=True)
            except Exception as e2:
                print(f"emergency checkpoint failed: {e2}", file=sys.stderr)
        return 1
    if eng.wait_checkpoint() != 0:
        print("warning: a checkpoint write failed", file=sys.stderr)
    if n and is_printer:
        print(f"\nsummary: {n} steps | avg MFU {sum_mfu / n * 100:.1f}% | avg {sum_tps / n:.3e} tokens/s | "
              f"arena {h.arena_bytes / 2**30:.2f} GiB/gpu | {eng.launches_per_step} kernel launches/step")
    if sink:
        sink.close()
    eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
