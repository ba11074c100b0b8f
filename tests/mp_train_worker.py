"""Worker for multi-GPU tests: trains a tiny config (configs/tiny_mp.cfg by default) for a few steps under a given parallel
layout and writes the loss curve (rank 0). Launched with torch.distributed.run."""
import argparse
import json
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--config", default="tiny_mp")
    ap.add_argument("--zero", type=int, default=1)
    ap.add_argument("--comm", default="baseline")
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--graph", type=int, default=0)
    ap.add_argument("--burst", type=int, default=0,
                    help="train on one fixed batch; enqueue this many optimizer steps between two synchronisations")
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    import torch
    from cai_b200.runtime.engine import Engine, synthetic_batch
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    text = (ROOT / "configs" / f"{a.config}.cfg").read_text()
    text += f"\ngpus_per_rack = {world}\ngpus_per_tray = {world}\ntp = {a.tp}\npp = {a.pp}\nep = {a.ep}\ncomm = {a.comm}\nzero_stage = {a.zero}\n"
    eng = Engine(config_text=text, rank=rank, world=world, local_rank=int(os.environ.get("LOCAL_RANK", rank)))
    m = eng.model
    dp = eng.hdr.dp
    dp_id = rank // (a.tp * a.pp)
    rows = eng.hdr.num_microbatches * m.microbatch
    losses = []
    if a.burst:
        # every step sees the same batch, so a run that synchronises after each step and a run that enqueues
        # `burst` steps back to back must read the same loss after the same number of steps
        tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows * dp, step=0, seed=11)
        tok, tgt = tok[dp_id * rows:(dp_id + 1) * rows].contiguous().pin_memory(), tgt[dp_id * rows:(dp_id + 1) * rows].contiguous().pin_memory()
        eng.load_batch(tok, tgt)
        for step in range(0, a.steps, a.burst):
            for _ in range(a.burst):
                eng.run_step()
            losses.append(eng.read_loss())
    for step in range(a.steps if not a.burst else 0):
        # the global batch is dp * rows sequences; each data-parallel replica takes its slice
        tok, tgt = synthetic_batch(m.vocab_size, m.seq_len, rows * dp, step=step % 2, seed=11)
        tok, tgt = tok[dp_id * rows:(dp_id + 1) * rows].contiguous().pin_memory(), tgt[dp_id * rows:(dp_id + 1) * rows].contiguous().pin_memory()
        if a.graph and step == 2:
            eng.use_graph(True)
        losses.append(eng.step(tok, tgt))
    last_stage_rank0 = (a.pp - 1) * a.tp
    if rank == last_stage_rank0:
        Path(a.out).write_text(json.dumps({"losses": losses, "world": world, "tp": a.tp, "pp": a.pp, "dp": dp,
                                           "comm": a.comm, "launches": eng.launches_per_step}))
    eng.close()
    import torch.distributed as dist
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
