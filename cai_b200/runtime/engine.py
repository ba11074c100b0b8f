"""Device engine: one rank's compiled plan, its arena and the native executor.

``Engine`` is the public training API: build it from a config (or from plan files the offline
compiler wrote), feed it pinned host batches with :meth:`Engine.step`, read the loss back. All
device work — kernels, NCCL calls, fused compute+collective kernels — is issued by the C++
executor in ``libcai_kernels.so``; Python only owns the arena allocation (one ``torch`` buffer),
parameter initialisation, batches and checkpoints.
"""
from __future__ import annotations

import ctypes
import os
import tempfile
from ctypes import c_char_p, c_float, c_int, c_size_t, c_ulonglong, c_void_p
from pathlib import Path

import torch

from .. import plan as planlib
from ..ops import _lib as klib

_TORCH_DTYPE = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16, 3: torch.uint8, 4: torch.uint8,
                5: torch.int32, 6: torch.uint8}


class TraceRec(ctypes.Structure):
    _fields_ = [("op_index", ctypes.c_uint32), ("kind", ctypes.c_uint16), ("stream", ctypes.c_uint16),
                ("start_s", ctypes.c_double), ("end_s", ctypes.c_double), ("bytes", ctypes.c_uint64),
                ("flops", ctypes.c_uint64)]


def _declare_runtime(L):
    if getattr(L, "_cai_rt_declared", False):
        return
    P, I = c_void_p, c_int
    L.cai_exec_create.argtypes = [ctypes.POINTER(P), P, c_size_t, P, ctypes.POINTER(P)]
    L.cai_exec_destroy.argtypes = [P]
    L.cai_exec_destroy.restype = None
    L.cai_nccl_unique_id.argtypes = [c_char_p, P]
    L.cai_exec_init_comm.argtypes = [P, c_char_p, I, P, P, I, I]
    L.cai_exec_stream.argtypes = [P, I]
    L.cai_exec_stream.restype = P
    L.cai_exec_tensor_ptr.argtypes = [P, I]
    L.cai_exec_tensor_ptr.restype = P
    L.cai_exec_launches.argtypes = [P]
    L.cai_exec_launches.restype = c_ulonglong
    L.cai_exec_step.argtypes = [P, I, c_float]
    L.cai_exec_sync.argtypes = [P]
    L.cai_exec_use_graph.argtypes = [P, I]
    L.cai_exec_trace_enable.argtypes = [P, I]
    L.cai_exec_nvtx_enable.argtypes = [P, I]
    L.cai_exec_trace_read.argtypes = [P, ctypes.POINTER(TraceRec), I]
    L.cai_exec_set_sm_limit.argtypes = [P, I]
    L.cai_exec_set_sm_limit.restype = None
    L._cai_rt_declared = True


def nccl_library_path() -> str:
    """The NCCL that torch itself loaded (so the executor's communicators share one library)."""
    try:
        import nvidia.nccl
        cand = Path(list(nvidia.nccl.__path__)[0]) / "lib" / "libnccl.so.2"
        if cand.exists():
            return str(cand)
    except Exception:
        pass
    return "libnccl.so.2"


def synthetic_batch(vocab, seq, rows, step, seed, rank_offset=0, out_tokens=None, out_targets=None):
    """Uniform-random token rows and their next-token targets (pinned int32 ``[rows, seq]``)."""
    g = torch.Generator(device="cpu")
    g.manual_seed((int(seed) * 1000003 + int(step)) * 4099 + int(rank_offset))
    s = torch.randint(0, vocab, (rows, seq + 1), generator=g, dtype=torch.int32)
    if out_tokens is None:
        out_tokens = torch.empty((rows, seq), dtype=torch.int32).pin_memory()
        out_targets = torch.empty((rows, seq), dtype=torch.int32).pin_memory()
    out_tokens.copy_(s[:, :-1])
    out_targets.copy_(s[:, 1:])
    return out_tokens, out_targets


class DeviceStatusError(RuntimeError):
    """A kernel of the step gave up on a bounded wait (or refused its arguments) and said so in the device
    status word; the step's results are not to be trusted."""

    def __init__(self, status):
        super().__init__(f"a kernel gave up on a bounded wait (device status {status})")
        self.status = status


class Engine:
    """Executes one rank's plan. See the module docstring."""

    def __init__(self, config=None, *, config_text=None, plan_path=None, topology_path=None, rank=None, world=None,
                 local_rank=None, graph=False, init_params=True, comm=None):
        self.rank = int(os.environ.get("RANK", 0)) if rank is None else rank
        self.world = int(os.environ.get("WORLD_SIZE", 1)) if world is None else world
        self.local_rank = int(os.environ.get("LOCAL_RANK", self.rank)) if local_rank is None else local_rank
        if not torch.cuda.is_available():
            raise RuntimeError("Engine needs a CUDA device; use cai_b200.plan.Simulator for GPU-free replay")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        self._tmp = None
        if plan_path is None:
            if config_text is None:
                config_text = Path(config).read_text()
            if comm is not None:
                config_text += f"\ncomm = {comm}\n"
            self.config_text = config_text
            self._tmp = tempfile.TemporaryDirectory(prefix="cai_plan_")
            planlib.compile_plans(config_text, self._tmp.name, ranks=(self.rank, self.rank + 1), version=2, text=True)
            plan_path = Path(self._tmp.name) / f"plan.rank{self.rank:06d}.bin"
            topology_path = Path(self._tmp.name) / "topology.bin"
        else:
            self.config_text = config_text
        self.plan = planlib.PlanFile(plan_path)
        if self.plan.hdr.version != 2:
            raise planlib.PlanError(f"{plan_path} is a cost-only (version 1) plan; compile with --exec")
        self.topology = planlib.read_topology(topology_path)
        self.topology_path = str(topology_path)
        th = planlib.fnv1a(bytes(self.topology))
        if th != self.plan.hdr.topology_hash:
            raise planlib.PlanError("plan was compiled for a different topology (hash mismatch)")
        if self.plan.hdr.world_size != self.world:
            raise planlib.PlanError(f"plan world_size {self.plan.hdr.world_size} != launched world {self.world}")
        self.hdr, self.model, self.train = self.plan.hdr, self.plan.model, self.plan.train
        self.named = self.plan.named_dict()

        L = klib.lib()
        _declare_runtime(L)
        self.L = L
        # the whole arena is ONE allocation; every tensor of the plan is an offset into it. A guard region
        # filled with a known pattern sits on either side (check_canaries()).
        G = self._GUARD
        self.arena = torch.empty(int(self.hdr.arena_bytes) + 1024 + 2 * G, dtype=torch.uint8, device=self.device)
        base = (self.arena.data_ptr() + G + 1023) & ~1023
        self._arena_shift = base - self.arena.data_ptr()
        self.arena_base = base
        self.arena.zero_()
        self.arena[:self._arena_shift].fill_(0xA5)
        self.arena[self._arena_shift + int(self.hdr.arena_bytes):].fill_(0xA5)
        # guard bytes between the class segments of the arena (the compiler leaves them uncovered)
        self._inner_guards = self._segment_gaps()
        for lo, hi in self._inner_guards:
            self.arena[self._arena_shift + lo:self._arena_shift + hi].fill_(0xA5)
        self.ex = c_void_p()
        # The six streams come from torch's pool: tensors touched on them stay valid for torch's
        # caching allocators after the executor is gone. compute_hi and comm_tp get high priority.
        self.streams = [torch.cuda.Stream(device=self.device, priority=-1 if s in (0, 2) else 0) for s in range(6)]
        handles = (c_void_p * 6)(*[c_void_p(s.cuda_stream) for s in self.streams])
        klib.check(L.cai_exec_create(ctypes.byref(self.ex), self.plan.raw, len(self.plan.raw), c_void_p(base), handles),
                   "exec_create")
        self.stream = self.streams[0]
        self.step_count = 0          # optimizer steps enqueued
        self.completed_steps = 0     # optimizer steps whose loss was read back without a device error
        self.device_fault = False    # a kernel reported an error: the arena may be half-updated
        self.lr = float(self.train.lr)
        self._init_comms()
        self.tokens_dev = self.view("@tokens")
        self.targets_dev = self.view("@targets")
        self.loss_dev = self.view("@loss")
        self.loss_host = torch.zeros(8, dtype=torch.float32).pin_memory()
        # one row per launch of the schedule (the compiler may launch several microbatches together)
        self.batch_rows, self.batch_cols = int(self.tokens_dev.shape[0]), int(self.tokens_dev.shape[1])
        with torch.cuda.stream(self.stream):
            klib.check(L.cai_rope_table(c_void_p(self.view("@rope_table").data_ptr()), self.model.seq_len,
                                        self.model.head_dim, float(self.train.rope_theta),
                                        c_void_p(self.stream.cuda_stream)), "rope_table")
        if init_params:
            self.init_parameters()
        if graph:
            self.use_graph(True)
        torch.cuda.synchronize(self.device)

    _GUARD = 4096

    def _segment_gaps(self):
        """Byte ranges of the arena that lie between the tensors of one class and the first tensor of the next:
        the guard words the compiler leaves at the end of every class segment."""
        ext = {}
        for t in self.plan.tensors:
            if t.nbytes == 0:
                continue
            lo, hi = ext.get(t.tclass, (1 << 62, 0))
            ext[t.tclass] = (min(lo, t.offset), max(hi, t.offset + t.nbytes))
        order = sorted(ext.values())
        gaps = []
        for (lo_a, hi_a), (lo_b, _) in zip(order, order[1:] + [(int(self.hdr.arena_bytes), 0)]):
            if lo_b > hi_a:
                gaps.append((int(hi_a), int(lo_b)))
        return gaps

    def check_canaries(self):
        """Debug aid: the guard bytes on both sides of the arena and between its class segments (parameters,
        gradients, optimizer state, activations, communication buffers, workspace) must still hold their pattern,
        i.e. no kernel wrote past the end of the tensors of one class. Synchronises the device."""
        torch.cuda.synchronize(self.device)
        head = self.arena[:self._arena_shift]
        tail = self.arena[self._arena_shift + int(self.hdr.arena_bytes):]
        bad = int((head != 0xA5).sum().item()) + int((tail != 0xA5).sum().item())
        if bad:
            raise RuntimeError(f"{bad} guard bytes around the arena were overwritten")
        for lo, hi in self._inner_guards:
            n = int((self.arena[self._arena_shift + lo:self._arena_shift + hi] != 0xA5).sum().item())
            if n:
                raise RuntimeError(f"{n} guard bytes between arena segments (offsets {lo}..{hi}) were overwritten")
        return True

    # ------------------------------------------------------------------ arena views
    def tensor_view(self, tid: int) -> torch.Tensor:
        t = self.plan.tensors[tid]
        rows, cols, ld = self.plan.shape(tid)
        dt = _TORCH_DTYPE[t.dtype]
        off = self._arena_shift + t.offset
        flat = self.arena[off:off + t.nbytes].view(dt)
        if ld == 0 or rows * ld != flat.numel():
            return flat
        return flat.view(rows, ld)[:, :cols]

    def view(self, name: str) -> torch.Tensor:
        return self.tensor_view(self.named[name].tensor)

    def param(self, name: str) -> torch.Tensor:
        if getattr(self, "zero3", False):
            raise RuntimeError("parameters are sharded (zero_stage = 3): a named tensor is only a place in a staging "
                               "buffer that holds it while its layer runs")
        return self.view(name)

    def grad(self, name: str) -> torch.Tensor:
        return self.tensor_view(self.named[name].grad)

    def parameter_names(self):
        return [k for k, v in self.named.items() if v.init_std >= 0]

    # ------------------------------------------------------------------ communicators
    def _init_comms(self):
        self.dist = None
        groups = [g for g in self.plan.groups if g.size > 1]
        if not groups:
            return
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group(backend="cpu:gloo,cuda:nccl", rank=self.rank, world_size=self.world,
                                    device_id=self.device)
        self.dist = dist
        store = dist.distributed_c10d._get_default_store()
        libpath = nccl_library_path().encode()
        for g in groups:
            members = planlib.group_members(self.config_text, g.kind, self.rank)
            me = members.index(self.rank)
            n_ids = 2 if g.kind in (planlib.GROUP_PP, planlib.GROUP_TP) else 1
            key = f"cai/nccl/{self.hdr.plan_hash:x}/{g.kind}/{g.color}"
            if me == 0:
                blob = b""
                for _ in range(n_ids):
                    buf = ctypes.create_string_buffer(128)
                    klib.check(self.L.cai_nccl_unique_id(libpath, buf), "nccl_unique_id")
                    blob += buf.raw
                store.set(key, blob)
            else:
                blob = store.get(key)
            id1 = ctypes.create_string_buffer(blob[:128], 128)
            id2 = ctypes.create_string_buffer(blob[128:256], 128) if n_ids == 2 else None
            klib.check(self.L.cai_exec_init_comm(self.ex, libpath, g.kind, id1, id2, len(members), me), "init_comm")
        self.peers = None
        if self.train.comm_mode:
            # fused compute+collective kernels address the other members' arenas directly
            from ..parallel import peers
            self.peers = peers.attach(self, groups, store)
            torch.cuda.synchronize(self.device)
            dist.barrier(device_ids=[self.local_rank])

    # ------------------------------------------------------------------ parameters
    def _global_shape_and_slice(self, name, rows, cols):
        """Global shape of a parameter and the index expression of this rank's shard."""
        m, tp = self.model, self.hdr.tp
        tp_id = self.rank % tp
        H, hd = m.hidden_size, m.head_dim
        base = name.split(".")[-1]
        if ".experts." in name:
            # local experts are a contiguous block of rows of the all-experts tensor
            # (under tensor parallelism the experts are spread over the tp x ep ranks of the expert group)
            ep = max(1, self.hdr.ep)
            ep_id = (self.rank // (self.hdr.tp * self.hdr.num_stages * self.hdr.cp)) % ep
            members, me = ep * tp, ep_id * tp + tp_id
            return (rows * members, cols), (slice(me * rows, (me + 1) * rows), slice(None))
        if base in ("embed", "lm_head"):
            return (m.vocab_size, H), (slice(tp_id * rows, (tp_id + 1) * rows), slice(None))
        if base == "wqkv":
            nh_l, nkv_l = m.num_heads // tp, m.num_kv_heads // tp
            q0, k0, v0 = 0, m.num_heads * hd, (m.num_heads + m.num_kv_heads) * hd
            idx = torch.cat([torch.arange(q0 + tp_id * nh_l * hd, q0 + (tp_id + 1) * nh_l * hd),
                             torch.arange(k0 + tp_id * nkv_l * hd, k0 + (tp_id + 1) * nkv_l * hd),
                             torch.arange(v0 + tp_id * nkv_l * hd, v0 + (tp_id + 1) * nkv_l * hd)])
            return ((m.num_heads + 2 * m.num_kv_heads) * hd, H), (idx, slice(None))
        if base == "wo":
            return (H, m.num_heads * hd), (slice(None), slice(tp_id * cols, (tp_id + 1) * cols))
        if base == "wgu":
            F, F_l = m.ffn_hidden, m.ffn_hidden // tp
            idx = torch.cat([torch.arange(tp_id * F_l, (tp_id + 1) * F_l), torch.arange(F + tp_id * F_l, F + (tp_id + 1) * F_l)])
            return (2 * F, H), (idx, slice(None))
        if base == "wd":
            return (H, m.ffn_hidden), (slice(None), slice(tp_id * cols, (tp_id + 1) * cols))
        return (rows, cols), (slice(None), slice(None))

    def init_parameters(self):
        """N(0, init_std) for matrices, ones for norm gains. Every rank draws the full tensor from a
        seed derived from the parameter's name and keeps its shard, so the model is the same for
        every parallel layout."""
        n_flat = int(self.plan.xhdr.param_elems)
        n_opt = int(self.plan.xhdr.opt_elems)
        master = self.view("@flat_master")
        dp, dp_id = self.hdr.dp, self.rank // (self.hdr.tp * self.hdr.num_stages * self.hdr.cp)
        # [0, n_rep) of the flat space is replicated over the data-parallel group (optimizer state
        # possibly sharded, n_shard elements per rank); [n_rep, n_flat) holds this rank's own experts,
        # whose state follows the shard in the optimizer buffers.
        split = self.named.get("@flat_split")
        n_rep = int(split.flat_off512) * 512 if split is not None else n_flat
        n_shard = int(split.rows) * 512 if split is not None else n_opt
        sharded = dp > 1 and n_shard < n_rep   # optimizer state split over the data-parallel group
        shard_lo = dp_id * n_shard if sharded else 0
        shard_hi = min(shard_lo + n_shard, n_rep) if sharded else n_rep
        pshard = self.view("@flat_param")
        self.zero3 = sharded and pshard.numel() < n_flat   # bf16 parameters sharded like the optimizer state
        with torch.cuda.stream(self.stream):
            self.view("@flat_m").zero_()
            self.view("@flat_v").zero_()
            master.zero_()
            for name, nt in self.named.items():
                if nt.init_std < 0:
                    continue
                w = self.tensor_view(nt.tensor)
                if nt.init_std == 0:
                    full = torch.ones((nt.rows, nt.cols), device=self.device, dtype=torch.float32)
                else:
                    gshape, idx = self._global_shape_and_slice(name, nt.rows, nt.cols)
                    g = torch.Generator(device=self.device)
                    g.manual_seed(planlib.fnv1a(name.encode(), int(self.train.seed) + 1) & 0x7FFFFFFFFFFFFFFF)
                    glob = torch.randn(gshape, generator=g, device=self.device, dtype=torch.float32) * nt.init_std
                    r, c = idx
                    if isinstance(r, torch.Tensor):
                        full = glob[r.to(self.device)][:, c]
                    else:
                        full = glob[r, c]
                    del glob
                if not self.zero3:
                    w.copy_(full.to(torch.bfloat16))
                # fp32 master copy of the part of this tensor that falls into this rank's optimizer shard
                lo = nt.flat_off512 * 512
                hi = lo + nt.rows * nt.cols
                if lo >= n_rep:
                    master[n_shard + lo - n_rep:n_shard + hi - n_rep].copy_(full.reshape(-1))
                    continue
                a, b = max(lo, shard_lo), min(hi, shard_hi)
                if a < b:
                    master[a - shard_lo:b - shard_lo].copy_(full.reshape(-1)[a - lo:b - lo])
                    if self.zero3:
                        pshard[a - shard_lo:b - shard_lo].copy_(full.reshape(-1)[a - lo:b - lo].to(torch.bfloat16))
        torch.cuda.synchronize(self.device)
        self._peer_barrier()

    def _peer_barrier(self):
        """Members read each other's parameter shards from the first kernel of a step (zero_stage = 3):
        nobody starts before every member has written its shard."""
        if getattr(self, "zero3", False) and self.dist is not None and self.dist.is_initialized():
            torch.cuda.synchronize(self.device)
            self.dist.barrier(device_ids=[self.local_rank])

    # ------------------------------------------------------------------ stepping
    def use_graph(self, on=True):
        klib.check(self.L.cai_exec_use_graph(self.ex, int(on)), "use_graph")

    def load_batch(self, tokens: torch.Tensor, targets: torch.Tensor):
        """Async host->device copy of one step's inputs (pinned int32 ``[grad_accum, microbatch*seq]``)."""
        with torch.cuda.stream(self.stream):
            self.tokens_dev.copy_(tokens.view(self.batch_rows, self.batch_cols), non_blocking=True)
            self.targets_dev.copy_(targets.view(self.batch_rows, self.batch_cols), non_blocking=True)
        return tokens.numel() * 4 + targets.numel() * 4

    def run_step(self, lr=None):
        """Enqueue one optimizer step on the batch already on the device."""
        self.step_count += 1
        klib.check(self.L.cai_exec_step(self.ex, self.step_count, float(self.lr if lr is None else lr)), "exec_step")

    def read_loss(self) -> float:
        """Device->host read of the step's mean loss (synchronises the step)."""
        with torch.cuda.stream(self.stream):
            self.loss_host.copy_(self.loss_dev.view(-1)[:8], non_blocking=True)
        klib.check(self.L.cai_exec_sync(self.ex), "exec_sync")
        st = klib.device_status(clear=True)
        if st != 0:
            self.device_fault = True
            raise DeviceStatusError(st)
        self.completed_steps = self.step_count
        return float(self.loss_host[0])

    def step(self, tokens, targets, lr=None) -> float:
        self.load_batch(tokens, targets)
        self.run_step(lr)
        return self.read_loss()

    def synchronize(self):
        klib.check(self.L.cai_exec_sync(self.ex), "exec_sync")

    @property
    def launches_per_step(self) -> int:
        return int(self.L.cai_exec_launches(self.ex))

    # ------------------------------------------------------------------ trace
    def debug_bounds(self, on=True):
        """Check every operand's extent against the plan's tensor table before each launch (slow path for debugging;
        ``CAI_DEBUG_BOUNDS=1`` in the environment switches it on from the start)."""
        self.L.cai_exec_set_debug.argtypes = [c_void_p, c_int]
        self.L.cai_exec_set_debug(self.ex, int(on))

    def nvtx(self, on=True):
        """One NVTX range per op of a replay, named by kernel, for timeline tools."""
        self.L.cai_exec_nvtx_enable(self.ex, int(on))

    def trace_step(self, tokens, targets):
        """Run one step with per-op CUDA events; returns a list of TraceRec with measured times."""
        self.L.cai_exec_use_graph(self.ex, 0)
        self.L.cai_exec_trace_enable(self.ex, 1)
        self.step(tokens, targets)
        buf = (TraceRec * len(self.plan.ops))()
        n = self.L.cai_exec_trace_read(self.ex, buf, len(buf))
        self.L.cai_exec_trace_enable(self.ex, 0)
        return [buf[i] for i in range(n)]

    @staticmethod
    def stream_stats(recs):
        """Measured per-stream occupancy and idle share of the main compute stream from one traced step.

        Returns ``(step_time_s, busy_s[6], bubble)``: busy is the summed duration of the ops of each of the six
        logical streams (the reference prints the same six columns from its cost model, tools/trainer.c:86-91);
        bubble is the time compute_hi spent without an op in flight between the first op of the step and the
        last one on any stream, over the step time (for a pipeline stage: fill, drain and hand-off waits)."""
        if not recs:
            return 0.0, [0.0] * 6, 0.0
        t0 = min(r.start_s for r in recs)
        t1 = max(r.end_s for r in recs)
        busy = [0.0] * 6
        for r in recs:
            busy[r.stream] += max(0.0, r.end_s - r.start_s)
        hi = sorted(((r.start_s, r.end_s) for r in recs if r.stream == 0))
        covered, cur_s, cur_e = 0.0, None, None
        for s, e in hi:
            if cur_e is None or s > cur_e:
                if cur_e is not None:
                    covered += cur_e - cur_s
                cur_s, cur_e = s, e
            else:
                cur_e = max(cur_e, e)
        if cur_e is not None:
            covered += cur_e - cur_s
        step = t1 - t0
        return step, busy, (1.0 - covered / step) if step > 0 else 0.0

    def abort_pending_waits(self):
        """Host-side lever of the watchdog: kernels of this device that sit in a bounded wait give up now."""
        klib.status_abort()

    # ------------------------------------------------------------------ checkpoint / resume
    # File layout (per rank): "<path>.<tag>.rank%06u" plus a rolling "<path>.latest.rank%06u". The
    # first 12 bytes are the reference's (u32 step, u64 plan_hash; src/runtime.c:244-262); a section
    # table follows with this rank's resident state: bf16 parameters, fp32 master / m / v shard,
    # step counter. The snapshot is copied device->host on the io stream into pinned buffers and the
    # file is written (temporary name + rename) by a background thread, so saving overlaps training.
    def save_checkpoint(self, path, tag="periodic", wait=False, roll_latest=True, state=True):
        """Snapshot this rank's parameters and optimizer state. ``roll_latest=False`` leaves the rolling
        "latest" file alone (a snapshot taken after a failed step must not replace the last good one);
        ``state=False`` writes the step counter only (nothing on the device is read)."""
        import threading
        # the previous writer may still be streaming the pinned buffers to disk: it has to finish before the
        # new device-to-host copies land in them
        prev = getattr(self, "_ckpt_thread", None)
        if prev is not None:
            prev.join()
            self._ckpt_thread = None
        host = {}
        done = None
        if state:
            sections = {"param": self.view("@flat_param"), "master": self.view("@flat_master"),
                        "m": self.view("@flat_m"), "v": self.view("@flat_v")}
            io = self.streams[5]
            io.wait_stream(self.stream)
            pinned = getattr(self, "_ckpt_pinned", {})
            with torch.cuda.stream(io):
                for k, t in sections.items():
                    buf = pinned.get(k)
                    if buf is None or buf.numel() != t.numel() or buf.dtype != t.dtype:
                        buf = torch.empty(t.shape, dtype=t.dtype).pin_memory()
                    buf.copy_(t, non_blocking=True)
                    host[k] = buf
            self._ckpt_pinned = host
            done = torch.cuda.Event()
            done.record(io)
            self.stream.wait_event(done)  # the next optimizer update must not overtake the snapshot
        # the step this state belongs to: the last one whose loss was read back without a device error
        step = self.completed_steps if not state or tag == "emergency" else self.step_count
        ph, rank = int(self.hdr.plan_hash), self.rank

        def write():
            import numpy as np
            if done is not None:
                done.synchronize()
            meta = np.array([step], dtype=np.int64)
            names = list(host) + ["meta"]
            arrs = [host[k].view(torch.uint8).numpy() if host[k].dtype != torch.bfloat16
                    else host[k].view(torch.int16).numpy().view(np.uint8) for k in host] + [meta.view(np.uint8)]
            n = len(names)
            c_names = (ctypes.c_char_p * n)(*[x.encode() for x in names])
            c_data = (c_void_p * n)(*[c_void_p(a.ctypes.data) for a in arrs])
            c_len = (ctypes.c_uint64 * n)(*[a.nbytes for a in arrs])
            rc = planlib.lib().cai_ckpt_write2(str(path).encode(), tag.encode(), rank, step, ph, n, c_names, c_data, c_len,
                                               1 if roll_latest else 0)
            self._ckpt_rc = rc

        self._ckpt_rc = 0
        th = threading.Thread(target=write, daemon=True)
        th.start()
        self._ckpt_thread = th
        if wait:
            th.join()
            if self._ckpt_rc != 0:
                raise IOError(f"checkpoint write failed ({self._ckpt_rc}) for {path}")

    def save_emergency_checkpoint(self, path):
        """What the trainer leaves behind after a failed step (the reference's "emergency" tag,
        tools/trainer.c:62-67). The rolling "latest" file is never touched. When a kernel reported an
        error (a bounded wait ran out) the device state may be half-updated, so only the number of the
        last completed step is recorded; otherwise the state is saved under the emergency tag."""
        try:
            clean = klib.device_status(clear=False) == 0 and not self.device_fault
        except Exception:
            clean = False
        self.save_checkpoint(path, "emergency", wait=True, roll_latest=False, state=clean)
        return clean

    def wait_checkpoint(self):
        th = getattr(self, "_ckpt_thread", None)
        if th is not None:
            th.join()
            self._ckpt_thread = None
        return getattr(self, "_ckpt_rc", 0)

    def load_checkpoint(self, path) -> bool:
        """Resume from "<path>.latest.rank..." (or the literal path). Returns False when there is
        nothing to resume from; raises when the checkpoint belongs to another plan."""
        import numpy as np
        L = planlib.lib()
        step, ph, nsec = ctypes.c_uint32(0), ctypes.c_uint64(0), ctypes.c_uint32(0)
        resolved = ctypes.create_string_buffer(1024)
        rc = L.cai_ckpt_probe(str(path).encode(), self.rank, ctypes.byref(step), ctypes.byref(ph), ctypes.byref(nsec),
                              resolved, len(resolved))
        if rc == 1:
            return False
        if rc != 0:
            raise IOError(f"cannot read checkpoint {path}")
        if ph.value != self.hdr.plan_hash:
            raise planlib.PlanError(f"checkpoint {resolved.value.decode()} belongs to plan {ph.value:016x}, "
                                    f"this plan is {int(self.hdr.plan_hash):016x}")
        targets = {"param": self.view("@flat_param"), "master": self.view("@flat_master"), "m": self.view("@flat_m"),
                   "v": self.view("@flat_v")}
        for i in range(nsec.value):
            name = ctypes.create_string_buffer(16)
            nbytes = ctypes.c_uint64(0)
            L.cai_ckpt_section(resolved.value, i, name, ctypes.byref(nbytes), None, 0)
            buf = np.empty(nbytes.value, dtype=np.uint8)
            rc = L.cai_ckpt_section(resolved.value, i, name, ctypes.byref(nbytes), c_void_p(buf.ctypes.data), buf.nbytes)
            if rc != 0:
                raise IOError(f"checkpoint section {i} unreadable")
            key = name.value.decode()
            if key == "meta":
                self.step_count = self.completed_steps = int(buf.view(np.int64)[0])
            elif key in targets:
                t = targets[key]
                src = torch.from_numpy(buf)
                if src.numel() != t.numel() * t.element_size():
                    raise planlib.PlanError(f"checkpoint section {key} has the wrong size")
                with torch.cuda.stream(self.stream):
                    t.view(torch.uint8).view(-1).copy_(src.to(self.device))
        self.synchronize()
        # every rank must resume from the same step: a rank whose newest file is older (or newer) than the
        # others' would train a model that no longer exists
        if self.dist is not None and self.dist.is_initialized() and self.world > 1:
            t = torch.tensor([self.step_count, -self.step_count], device=self.device, dtype=torch.int64)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            hi, lo = int(t[0].item()), -int(t[1].item())
            if hi != lo:
                raise planlib.PlanError(f"ranks resume from different steps ({lo}..{hi}): restore a common checkpoint")
        self._peer_barrier()
        return True

    # ------------------------------------------------------------------ metrics
    def tokens_per_step(self) -> int:
        return int(self.hdr.global_tokens_per_step)

    def mfu(self, step_time_s: float, peak_flops: float = None) -> float:
        peak = peak_flops or self.topology.gpu_flops_bf16
        useful = self.hdr.global_tokens_per_step * self.hdr.flops_per_token_useful / self.hdr.world_size
        return useful / (peak * step_time_s) if step_time_s > 0 else 0.0

    def close(self):
        self.wait_checkpoint()
        if getattr(self, "ex", None) and getattr(self, "peers", None) and self.dist is not None and self.dist.is_initialized():
            # nobody may unmap or free an arena while a peer's kernel can still touch it
            torch.cuda.synchronize(self.device)
            try:
                self.dist.barrier(device_ids=[self.local_rank])
            except Exception:
                pass
        if getattr(self, "ex", None):
            self.L.cai_exec_destroy(self.ex)
            self.ex = None
        if getattr(self, "peers", None):
            self.peers.close()
            self.peers = None
        if self._tmp is not None:
            self._tmp.cleanup()
            self._tmp = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
