"""Device trainer: one process == one GPU rank.

    python -m cai_b200.trainer <plan.bin> <topology.bin> [--steps N] [--ckpt PATH] [--ckpt-every K]
                               [--trace CSV] [--graph] [--nvtx] [--jsonl FILE]
                               [--data TOKENS] [--lr-warmup N] [--lr-decay cosine|linear]
                               [--step-timeout S] [--peer-timeout S] [--fail-at STEP]
    python -m cai_b200.trainer --config configs/x.cfg [...]        (compiles this rank's plan first)

Same command line, table and checkpoint naming as the reference's ``trainer`` (tools/trainer.c),
but the plan is executed on the GPU: real kernels, measured step time / MFU / tokens/s and a loss
column. The last step of a run is replayed with one CUDA-event pair per op, which gives the summary's
measured per-stream occupancy (the reference prints its cost model's, tools/trainer.c:86-91), the
measured idle share of the compute stream next to the pipeline-bubble formula, and the op timeline of
``--trace``. MFU is printed against the peak in ``topology.bin`` and, when ``MEASURED_PEAKS.json``
sits at the repository root, against the measured sustained bf16 throughput.

Failure handling: every step runs under a watchdog (``--step-timeout``); between steps every rank
publishes its progress in the job store and checks its peers' (``--peer-timeout``). A failed step, a
silent peer or an overrun ends the run with exit code 1 after an "emergency" checkpoint, as the
reference does (tools/trainer.c:62-67): the state when the device is clean, otherwise only the number
of the last completed step; the rolling "latest" checkpoint is never replaced by it.

Rank and world size come from RANK / WORLD_SIZE / LOCAL_RANK (``launch.sh`` or
``torch.distributed.run`` set them). Data is a synthetic uniform-random token stream, a different
slice per data-parallel replica, or with ``--data`` windows of a token file (``cai_b200/utils/data.py``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

import torch

from . import plan as planlib
from .runtime.engine import Engine, synthetic_batch
from .utils.data import TokenBatches
from .utils.health import Heartbeat, RankFailure, Watchdog
from .utils.schedule import lr_at

ROOT = Path(__file__).resolve().parent.parent


def measured_peak_flops():
    """Sustained bf16 matmul throughput measured on this pool (driver-written file), or None."""
    f = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(f.read_text())["bf16_tflops_sustained"]) * 1e12
    except Exception:
        return None


def write_trace_json(path, recs, rank=0):
    """The measured timeline in the Trace Event format (chrome://tracing, Perfetto): one track per logical stream."""
    ev = [{"ph": "M", "pid": rank, "tid": s, "name": "thread_name", "args": {"name": planlib.STREAMS[s]}} for s in range(6)]
    ev += [{"ph": "X", "pid": rank, "tid": r.stream, "name": planlib.OP_NAMES[r.kind], "ts": r.start_s * 1e6,
            "dur": (r.end_s - r.start_s) * 1e6, "args": {"op": r.op_index, "bytes": r.bytes, "flops": r.flops}} for r in recs]
    with open(path, "w") as f:
        json.dump({"displayTimeUnit": "ms", "traceEvents": ev}, f)


def write_trace_csv(path, recs):
    if str(path).endswith(".json"):
        return write_trace_json(path, recs)
    with open(path, "w") as f:
        f.write("op_index,kind,stream,start_us,end_us,dur_us,bytes,flops\n")
        for r in recs:
            f.write(f"{r.op_index},{planlib.OP_NAMES[r.kind]},{planlib.STREAMS[r.stream]},{r.start_s * 1e6:.4f},"
                    f"{r.end_s * 1e6:.4f},{(r.end_s - r.start_s) * 1e6:.4f},{r.bytes},{r.flops}\n")


def predicted_step_time(eng, rank):
    """Step time the calibrated pricing backend predicts for the running plan. A pipelined job is replayed with all
    of its stages together (the sibling stages' plans are compiled from the configuration when it is known); otherwise,
    and for a single stage, this rank's plan alone."""
    h = eng.hdr
    if h.num_stages > 1 and eng.config_text:
        import tempfile
        stride = h.tp * max(1, h.cp)
        base = rank - h.pipeline_stage * stride
        with tempfile.TemporaryDirectory(prefix="cai_predict_") as tmp:
            for s in range(h.num_stages):
                planlib.compile_plans(eng.config_text, tmp, ranks=(base + s * stride, base + s * stride + 1), version=2, text=True)
            paths = [Path(tmp) / f"plan.rank{base + s * stride:06d}.bin" for s in range(h.num_stages)]
            return planlib.pipeline_replay(paths, Path(tmp) / "topology.bin", backend="calibrated")["step_time_s"]
    sim = planlib.Simulator(eng.plan.path, eng.topology_path, rank=rank, backend="calibrated")
    try:
        return sim.step().step_time_s
    finally:
        sim.close()


def main(argv=None):
    ap = argparse.ArgumentParser(prog="cai_b200.trainer")
    ap.add_argument("plan", nargs="?")
    ap.add_argument("topology", nargs="?")
    ap.add_argument("--config")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--ckpt")
    ap.add_argument("--ckpt-every", type=int, default=0)
    ap.add_argument("--trace", help="write the last step's measured op timeline: CSV (reference schema), or Trace Event JSON for chrome://tracing / Perfetto when the path ends in .json")
    ap.add_argument("--graph", action="store_true")
    ap.add_argument("--nvtx", action="store_true", help="NVTX range per op, named by kernel (for timeline tools)")
    ap.add_argument("--jsonl")
    ap.add_argument("--comm", choices=["fused", "baseline"])
    ap.add_argument("--data", help="token file (raw uint16 / uint32 ids, or .npy) to train on; default: synthetic tokens")
    ap.add_argument("--data-dtype", choices=["uint16", "uint32"], default=None, help="id width of a raw --data file (default uint16)")
    ap.add_argument("--lr-warmup", type=int, default=0, help="steps of linear learning-rate warm-up")
    ap.add_argument("--lr-decay", choices=["none", "cosine", "linear"], default="none", help="decay after the warm-up")
    ap.add_argument("--lr-total", type=int, default=0, help="step at which the decay ends (default: --steps)")
    ap.add_argument("--lr-min-ratio", type=float, default=0.1, help="final rate as a share of the configured one")
    ap.add_argument("--step-timeout", type=float, default=600.0, help="watchdog deadline of one step in seconds (0 = off)")
    ap.add_argument("--peer-timeout", type=float, default=120.0, help="how long to wait for the other ranks between steps (0 = off)")
    ap.add_argument("--fail-at", type=int, default=-1, help="raise in the step callback at this step (host-side fault injection)")
    ap.add_argument("--no-stream-stats", action="store_true", help="do not replay the last step with per-op events")
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
    peak_measured = measured_peak_flops()
    sum_mfu = sum_tps = 0.0
    n = 0
    start_ev, stop_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first = eng.step_count
    if a.nvtx:
        eng.nvtx(True)

    # ---- failure detection (host side): heartbeat between steps, watchdog around each step
    hb = None
    if eng.dist is not None and eng.world > 1 and a.peer_timeout > 0:
        hb = Heartbeat(eng.dist.distributed_c10d._get_default_store(), rank, eng.world, prefix=f"cai/hb/{int(h.plan_hash):x}")
        hb.beat(first)

    def emergency(reason):
        print(f"step {eng.step_count} failed: {reason}", file=sys.stderr)
        if a.ckpt:
            try:
                with_state = eng.save_emergency_checkpoint(a.ckpt)
                print(f"[cai WARN] emergency checkpoint written ({'state of' if with_state else 'number of'} step "
                      f"{eng.completed_steps})", file=sys.stderr)
            except Exception as e2:  # noqa: BLE001
                print(f"emergency checkpoint failed: {e2}", file=sys.stderr)

    def on_overrun():
        # runs in the watchdog thread while the main thread may be blocked in a synchronise: make the waiting
        # kernels give up, record the last completed step (no device access) and end the process
        print(f"step {eng.step_count} overran its deadline of {a.step_timeout:.0f} s", file=sys.stderr)
        try:
            eng.abort_pending_waits()
        except Exception:  # noqa: BLE001
            pass
        if a.ckpt:
            try:
                eng.device_fault = True
                eng.save_checkpoint(a.ckpt, "emergency", wait=True, roll_latest=False, state=False)
            except Exception as e2:  # noqa: BLE001
                print(f"emergency checkpoint failed: {e2}", file=sys.stderr)
        sys.stderr.flush()
        os._exit(1)

    data = None
    if a.data:
        data = TokenBatches(a.data, m.vocab_size, m.seq_len, rows * h.dp, eng.train.seed, dp=h.dp, dp_id=dp_id, dtype=a.data_dtype)
        if is_printer:
            print(f"data: {len(data.tokens):,} tokens from {a.data}, {rows * h.dp} windows of {m.seq_len} per step")
    base_lr = float(eng.lr)
    scheduled = a.lr_warmup > 0 or a.lr_decay != "none"
    dog = Watchdog(a.step_timeout, on_overrun) if a.step_timeout > 0 else None
    stream_line = None
    try:
        for step in range(first, a.steps):
            straggler = None
            if hb is not None:
                # raises RankFailure naming the silent ranks; a peer that keeps everyone waiting for a large share
                # of a step is reported as a straggler
                waited, last_rank = hb.check(step, timeout=a.peer_timeout)
                if n and waited > max(0.25 * (h.global_tokens_per_step * n / sum_tps), 0.05):
                    straggler = {"rank": last_rank, "waited_s": waited}
                    print(f"rank {rank}: waited {waited * 1e3:.0f} ms for rank {last_rank} before step {step}", file=sys.stderr)
            if data is not None:
                tok, tgt = data.get(step)       # prefetched into pinned memory; a function of (seed, step) only
            else:
                tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows * h.dp, step=step, seed=eng.train.seed)
                tok = tok[dp_id * rows:(dp_id + 1) * rows].contiguous().pin_memory()
                tgt = tgt[dp_id * rows:(dp_id + 1) * rows].contiguous().pin_memory()
            if a.graph and step == first + 1:
                eng.use_graph(True)
            if step == a.fail_at:
                raise RuntimeError("injected failure (--fail-at)")
            if scheduled:
                eng.lr = lr_at(step, base_lr, a.lr_warmup, a.lr_total or a.steps, a.lr_decay, a.lr_min_ratio)
            last = step == a.steps - 1
            traced = last and (a.trace or not a.no_stream_stats)
            if dog:
                dog.arm()
            if traced:
                # the last step runs with one event pair per op: step time, per-stream occupancy and the idle
                # share of the compute stream come from the same timeline
                recs = eng.trace_step(tok, tgt)
                loss = float(eng.loss_host[0])
                dt, busy, idle = Engine.stream_stats(recs)
                stream_line = (busy, idle)
                if a.trace:
                    write_trace_csv(a.trace, recs)
                    if is_printer:
                        print(f"wrote op timeline to {a.trace}")
            else:
                eng.load_batch(tok, tgt)
                with torch.cuda.stream(eng.stream):
                    start_ev.record()
                eng.run_step()
                with torch.cuda.stream(eng.stream):
                    stop_ev.record()
                loss = eng.read_loss()
                dt = start_ev.elapsed_time(stop_ev) * 1e-3
            if dog:
                dog.disarm()
            if hb is not None:
                hb.beat(step + 1)
            tps = h.global_tokens_per_step / dt
            mfu = eng.mfu(dt)
            if is_printer:
                print(f"{step:4d} | {dt * 1e3:7.2f} ms| {bubble * 100:5.1f}% | {mfu * 100:5.1f}% | {tps:9.2e} | "
                      f"{tps / h.world_size:9.1f} | {loss:7.4f}", flush=True)
                if sink:
                    rec = {"step": step, "step_time_s": dt, "mfu": mfu, "tokens_per_s": tps, "loss": loss, "time": time.time(),
                           "bubble_formula": bubble}
                    if peak_measured:
                        rec["mfu_vs_measured_peak"] = eng.mfu(dt, peak_measured)
                    if straggler:
                        rec["straggler"] = straggler
                    if scheduled:
                        rec["lr"] = eng.lr
                    if traced:
                        rec["stream_busy_ms"] = {planlib.STREAMS[i]: busy[i] * 1e3 for i in range(6)}
                        rec["bubble_measured"] = idle
                        rec["traced"] = True
                    sink.write(json.dumps(rec) + "\n")
                    sink.flush()
            if not traced:      # the traced step pays for its events; it stays out of the averages
                sum_mfu += mfu
                sum_tps += tps
                n += 1
            if ckpt_every and a.ckpt and eng.step_count % ckpt_every == 0:
                eng.save_checkpoint(a.ckpt, "periodic")
    except RankFailure as e:
        emergency(f"peers silent: {e}")
        return 1
    except Exception as e:  # a failed step leaves an emergency checkpoint behind, like the reference
        emergency(e)
        return 1
    finally:
        if dog:
            dog.close()
        if data is not None:
            data.close()
    if eng.wait_checkpoint() != 0:
        print("warning: a checkpoint write failed", file=sys.stderr)
    if is_printer and (n or stream_line):
        if n:
            line = (f"\nsummary: {n} steps | avg MFU {sum_mfu / n * 100:.1f}% of {eng.topology.gpu_flops_bf16 / 1e15:.2f} PF")
            if peak_measured:
                line += f" ({eng.mfu(h.global_tokens_per_step / (sum_tps / n), peak_measured) * 100:.1f}% of measured {peak_measured / 1e12:.0f} TF)"
            line += (f" | avg {sum_tps / n:.3e} tokens/s | arena {h.arena_bytes / 2**30:.2f} GiB/gpu | "
                     f"{eng.launches_per_step} kernel launches/step")
            print(line)
        if n:
            # what the calibrated pricing backend predicts for this rank's plan, next to what was measured
            try:
                predicted = predicted_step_time(eng, rank)
                measured = h.global_tokens_per_step / (sum_tps / n)
                print(f"calibrated model: {predicted * 1e3:.2f} ms/step predicted, {measured * 1e3:.2f} measured "
                      f"(measured / predicted = {measured / predicted:.2f})")
            except Exception as e:  # the prediction is a courtesy; a run never fails over it
                print(f"calibrated model: no prediction ({e})", file=sys.stderr)
        if stream_line:
            busy, idle = stream_line
            print("per-stream occupancy (ms), measured on the last step: " +
                  " ".join(f"{planlib.STREAMS[i]}={busy[i] * 1e3:.2f}" for i in range(6)))
            print(f"compute stream idle {idle * 100:.1f}% of the step (measured); pipeline bubble by formula {bubble * 100:.1f}%")
    if sink:
        sink.close()
    eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
