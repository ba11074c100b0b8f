"""Move a checkpoint from one parallel layout to another (no GPU involved).

A checkpoint is per rank: the rank's slice of every parameter, and its shard of the fp32 master weights and AdamW
moments, in the order of the plan's flat parameter space. ``plan_recover`` (like the reference's, tools/plan_recover.c)
regenerates the plan of a failed rank for the SAME layout; this tool covers the other recovery: continue on a different
number of GPUs or with a different tensor / pipeline / data / expert split. It compiles the plans of both layouts, rebuilds
every parameter's global master / m / v tensor from the source ranks' files (undoing the tensor-parallel row / column
splits, the expert blocks, the pipeline stages and the data-parallel optimizer shards) and cuts them again for the
destination ranks. bf16 parameters are the rounded master weights, as after every optimizer step.

    python -m cai_b200.utils.reshard --src-config a.cfg --src ckpt/run --dst-config b.cfg --dst ckpt/run_b

The whole optimizer state is held in host memory while it is rearranged (12 bytes per parameter).
"""
from __future__ import annotations

import argparse
import ctypes
import tempfile
from ctypes import c_char_p, c_void_p
from pathlib import Path

import numpy as np
import torch

from .. import plan as planlib

STATE = ("master", "m", "v")


def global_slice(name, rows, cols, model, tp, tp_id, ep, ep_id):
    """Global shape of a parameter and the (row index, column index) of one rank's part of it: the inverse of how a
    rank cuts its shard out of the full tensor when it initialises (same rules as ``Engine._global_shape_and_slice``)."""
    H, hd = model.hidden_size, model.head_dim
    base = name.split(".")[-1]
    full = slice(None)
    if ".experts." in name:
        members, me = max(1, ep) * tp, ep_id * tp + tp_id
        return (rows * members, cols), (slice(me * rows, (me + 1) * rows), full)
    if base in ("embed", "lm_head"):
        return (model.vocab_size, H), (slice(tp_id * rows, (tp_id + 1) * rows), full)
    if base == "wqkv":
        nh_l, nkv_l = model.num_heads // tp, model.num_kv_heads // tp
        q0, k0, v0 = 0, model.num_heads * hd, (model.num_heads + model.num_kv_heads) * hd
        idx = np.concatenate([np.arange(q0 + tp_id * nh_l * hd, q0 + (tp_id + 1) * nh_l * hd),
                              np.arange(k0 + tp_id * nkv_l * hd, k0 + (tp_id + 1) * nkv_l * hd),
                              np.arange(v0 + tp_id * nkv_l * hd, v0 + (tp_id + 1) * nkv_l * hd)])
        return ((model.num_heads + 2 * model.num_kv_heads) * hd, H), (idx, full)
    if base == "wo":
        return (H, model.num_heads * hd), (full, slice(tp_id * cols, (tp_id + 1) * cols))
    if base == "wgu":
        F, F_l = model.ffn_hidden, model.ffn_hidden // tp
        idx = np.concatenate([np.arange(tp_id * F_l, (tp_id + 1) * F_l), np.arange(F + tp_id * F_l, F + (tp_id + 1) * F_l)])
        return (2 * F, H), (idx, full)
    if base == "wd":
        return (H, model.ffn_hidden), (full, slice(tp_id * cols, (tp_id + 1) * cols))
    return (rows, cols), (full, full)      # replicated over the tensor-parallel group (norm gains, router weights)


class RankLayout:
    """What one rank of a layout holds: its coordinates and where its parameters sit in the flat space."""

    def __init__(self, pf: planlib.PlanFile, rank: int):
        h = pf.hdr
        self.rank, self.plan_hash = rank, int(h.plan_hash)
        self.tp, self.pp, self.dp, self.ep = int(h.tp), int(h.num_stages), int(h.dp), max(1, int(h.ep))
        self.stage, self.tp_id = int(h.pipeline_stage), rank % int(h.tp)
        self.dp_id = rank // (self.tp * self.pp * max(1, int(h.cp)))
        self.ep_id = self.dp_id % self.ep
        self.model = pf.model
        named = pf.named_dict()
        self.n_flat, self.n_opt = int(pf.xhdr.param_elems), int(pf.xhdr.opt_elems)
        split = named.get("@flat_split")
        self.n_rep = int(split.flat_off512) * 512 if split is not None else self.n_flat
        self.n_shard = int(split.rows) * 512 if split is not None else self.n_opt
        self.sharded = self.dp > 1 and self.n_shard < self.n_rep
        self.shard_lo = self.dp_id * self.n_shard if self.sharded else 0
        self.shard_hi = min(self.shard_lo + self.n_shard, self.n_rep) if self.sharded else self.n_rep
        self.param_elems = int(pf.tensors[named["@flat_param"].tensor].nbytes) // 2   # < n_flat under ZeRO-3
        self.params = [(n.name.decode(), int(n.flat_off512) * 512, int(n.rows), int(n.cols))
                       for n in pf.named if n.init_std >= 0 and not n.name.startswith(b"@")]

    def slice_of(self, name, rows, cols):
        return global_slice(name, rows, cols, self.model, self.tp, self.tp_id, self.ep, self.ep_id)


def layout_of(config_path, workdir=None):
    """Compile the executable plans of a configuration and describe every rank."""
    text = Path(config_path).read_text()
    world = planlib.describe(text)["world_size"]
    with tempfile.TemporaryDirectory(dir=workdir) as tmp:
        planlib.compile_plans(text, tmp, ranks=(0, world), version=2, text=True)
        return [RankLayout(planlib.PlanFile(Path(tmp) / f"plan.rank{r:06d}.bin"), r) for r in range(world)]


def read_rank(path, rank):
    """Sections of one rank's checkpoint file (``<path>.latest.rankNNNNNN`` or the literal path) as numpy arrays."""
    L = planlib.lib()
    step, ph, nsec = ctypes.c_uint32(0), ctypes.c_uint64(0), ctypes.c_uint32(0)
    resolved = ctypes.create_string_buffer(1024)
    rc = L.cai_ckpt_probe(str(path).encode(), rank, ctypes.byref(step), ctypes.byref(ph), ctypes.byref(nsec), resolved, len(resolved))
    if rc != 0:
        raise IOError(f"no readable checkpoint for rank {rank} under {path}")
    out = {"plan_hash": ph.value}
    for i in range(nsec.value):
        name = ctypes.create_string_buffer(16)
        nbytes = ctypes.c_uint64(0)
        L.cai_ckpt_section(resolved.value, i, name, ctypes.byref(nbytes), None, 0)
        buf = np.empty(nbytes.value, dtype=np.uint8)
        if L.cai_ckpt_section(resolved.value, i, name, ctypes.byref(nbytes), c_void_p(buf.ctypes.data), buf.nbytes) != 0:
            raise IOError(f"{resolved.value.decode()}: section {i} unreadable (checksum)")
        key = name.value.decode()
        if key == "meta":
            out["step"] = int(buf.view(np.int64)[0])
        elif key in STATE:
            out[key] = buf.view(np.float32)
    return out


def gather_global(layout, read):
    """Global master / m / v tensor of every parameter from the ranks of ``layout``. ``read(rank)`` returns that rank's
    sections (``read_rank`` bound to a path). Returns ``(state, step)`` with ``state[name][key]`` a float32 array."""
    state, step = {}, None
    groups = {}
    for rl in layout:
        groups.setdefault((rl.stage, rl.tp_id), []).append(rl)
    for (_, _), ranks in sorted(groups.items()):
        ranks.sort(key=lambda r: r.dp_id)
        files = {rl.rank: read(rl.rank) for rl in ranks}
        for f in files.values():
            if f["plan_hash"] != ranks[0].plan_hash:
                raise planlib.PlanError("checkpoint does not belong to the source configuration (plan hash)")
            if step is None:
                step = f["step"]
            elif f["step"] != step:
                raise planlib.PlanError(f"source ranks are at different steps ({step} and {f['step']})")
        first = ranks[0]
        # the replicated part of the flat space: data-parallel ranks own consecutive shards of the optimizer state
        rep = {k: np.zeros(first.n_rep, dtype=np.float32) for k in STATE}
        for rl in (ranks if first.sharded else ranks[:1]):
            n = rl.shard_hi - rl.shard_lo
            for k in STATE:
                rep[k][rl.shard_lo:rl.shard_hi] = files[rl.rank][k][:n]
        for name, lo, rows, cols in first.params:
            if lo >= first.n_rep:
                continue
            gshape, (ri, ci) = first.slice_of(name, rows, cols)
            replicated = isinstance(ri, slice) and ri == slice(None) and ci == slice(None)
            if replicated and first.tp_id != 0:
                continue
            ent = state.setdefault(name, {k: np.zeros(gshape, dtype=np.float32) for k in STATE})
            for k in STATE:
                ent[k][ri, ci] = rep[k][lo:lo + rows * cols].reshape(rows, cols)
        # this rank's own experts follow the shard in its optimizer buffers
        for rl in ranks:
            for name, lo, rows, cols in rl.params:
                if lo < rl.n_rep:
                    continue
                gshape, (ri, ci) = rl.slice_of(name, rows, cols)
                ent = state.setdefault(name, {k: np.zeros(gshape, dtype=np.float32) for k in STATE})
                a = rl.n_shard + lo - rl.n_rep
                for k in STATE:
                    ent[k][ri, ci] = files[rl.rank][k][a:a + rows * cols].reshape(rows, cols)
    return state, step


def rank_sections(rl: RankLayout, state, step):
    """Checkpoint sections of one destination rank cut out of the global state."""
    flat = {k: np.zeros(rl.n_flat, dtype=np.float32) for k in STATE}
    for name, lo, rows, cols in rl.params:
        gshape, (ri, ci) = rl.slice_of(name, rows, cols)
        ent = state.get(name)
        if ent is None or ent["master"].shape != tuple(gshape):
            raise planlib.PlanError(f"parameter {name} of the destination has no counterpart of shape {gshape} in the source")
        for k in STATE:
            flat[k][lo:lo + rows * cols] = ent[k][ri, ci].reshape(-1)
    out = {}
    n = rl.shard_hi - rl.shard_lo
    tail = rl.n_flat - rl.n_rep
    for k in STATE:
        sec = np.zeros(rl.n_opt, dtype=np.float32)
        sec[:n] = flat[k][rl.shard_lo:rl.shard_hi]
        if tail:
            sec[rl.n_shard:rl.n_shard + tail] = flat[k][rl.n_rep:]
        out[k] = sec
    bf = torch.from_numpy(flat["master"]).to(torch.bfloat16)          # what AdamW leaves in the bf16 parameters
    if rl.param_elems < rl.n_flat:                                    # ZeRO-3: the rank keeps its shard only
        part = torch.zeros(rl.param_elems, dtype=torch.bfloat16)
        part[:n] = bf[rl.shard_lo:rl.shard_hi]
        bf = part
    out["param"] = bf.view(torch.int16).numpy()
    out["meta"] = np.array([step], dtype=np.int64)
    return out


def write_rank(path, tag, rl: RankLayout, sections, step):
    names = ["param", "master", "m", "v", "meta"]
    arrs = [np.ascontiguousarray(sections[k]).view(np.uint8) for k in names]
    n = len(names)
    c_names = (c_char_p * n)(*[x.encode() for x in names])
    c_data = (c_void_p * n)(*[c_void_p(a.ctypes.data) for a in arrs])
    c_len = (ctypes.c_uint64 * n)(*[a.nbytes for a in arrs])
    rc = planlib.lib().cai_ckpt_write2(str(path).encode(), tag.encode(), rl.rank, step, rl.plan_hash, n, c_names, c_data, c_len, 1)
    if rc != 0:
        raise IOError(f"cannot write {path} for rank {rl.rank} ({rc})")


def reshard(src_config, src_path, dst_config, dst_path, tag="resharded"):
    """Read the checkpoint ``src_path`` of the layout ``src_config`` and write it for ``dst_config`` under ``dst_path``.
    Returns ``(step, number of parameters moved, destination ranks)``."""
    src, dst = layout_of(src_config), layout_of(dst_config)
    state, step = gather_global(src, lambda r: read_rank(src_path, r))
    # The LM head is tied to the embedding only in unpipelined layouts (tie_embeddings = 1 and pp = 1): going from tied to
    # untied the head starts as a copy of the embedding (same model); going back is possible only while they are equal.
    dst_names = {name for rl in dst for name, _, _, _ in rl.params}
    if "lm_head" in dst_names and "lm_head" not in state and "embed" in state:
        state["lm_head"] = {k: state["embed"][k].copy() for k in STATE}
    if "lm_head" in state and "lm_head" not in dst_names and "embed" in state:
        if not np.array_equal(state["lm_head"]["master"], state["embed"]["master"]):
            raise planlib.PlanError("the destination ties the LM head to the embedding, but the source trained them as two "
                                    "tensors: set tie_embeddings = 0 in the destination configuration")
    for rl in dst:
        write_rank(dst_path, tag, rl, rank_sections(rl, state, step), step)
    return step, sum(int(np.prod(e["master"].shape)) for e in state.values()), len(dst)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--src-config", required=True)
    ap.add_argument("--src", required=True, help="checkpoint path prefix of the source run (as given to --ckpt)")
    ap.add_argument("--dst-config", required=True)
    ap.add_argument("--dst", required=True, help="checkpoint path prefix to write for the destination layout")
    a = ap.parse_args(argv)
    step, n, ranks = reshard(a.src_config, a.src, a.dst_config, a.dst)
    print(f"step {step}: {n} parameters (master, m, v) rearranged for {ranks} ranks -> {a.dst}.latest.rank*")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
