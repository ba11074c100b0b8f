"""Python face of the offline compiler (``libcai_host.so``): compile configs into plan files,
describe a decomposition, verify a whole cluster, and read plan files back as ctypes structures.

The binary layouts mirror ``csrc/plan/formats.h``; version-1 files are byte-compatible with the
reference project (include/cai_plan.h, include/cai_topology.h).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, c_char, c_char_p, c_double, c_float, c_int, c_int32, c_size_t, c_uint16,
                    c_uint32, c_uint64, c_void_p)
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libcai_host.so"
_lib = None

PLAN_MAGIC = 0x50494143
TOPO_MAGIC = 0x504F5443
EXEC_MAGIC = 0x58494143

STREAMS = ["compute_hi", "compute_lo", "comm_tp", "comm_pp", "comm_dp", "io"]
OP_NAMES = ["gemm", "attn_fwd", "attn_bwd", "rmsnorm", "swiglu", "elementwise", "reduce_scatter", "all_gather",
            "all_reduce", "all_to_all", "pipe_send", "pipe_recv", "optimizer", "event_record", "event_wait",
            "gemm_rs", "ag_gemm", "rs_adamw", "fsdp_ag_gemm", "moe_dispatch_gemm", "moe_gemm_combine"]
TCLASSES = ["param", "grad", "optstate", "activation", "comm", "workspace"]
DTYPES = ["fp32", "bf16", "fp16", "fp8e4m3", "fp8e5m2", "int32", "uint8"]
DTYPE_SIZE = [4, 2, 2, 1, 1, 4, 1]
GROUP_TP, GROUP_DP, GROUP_PP, GROUP_EP = 0, 1, 2, 3
# kernel ids of the execution section (csrc/plan/formats.h, enum KernelId)
KERNEL_NAMES = ["none", "embed_fwd", "embed_bwd", "rmsnorm_fwd", "rmsnorm_bwd", "gemm", "rope", "attn_fwd", "attn_bwd",
                "swiglu_fwd", "swiglu_bwd", "cross_entropy", "adamw", "zero", "nccl_all_reduce", "nccl_reduce_scatter",
                "nccl_all_gather", "nccl_all_to_all", "nccl_send", "nccl_recv", "gemm_rs", "ag_gemm", "rs_adamw",
                "fsdp_ag_gemm", "moe_route", "moe_dispatch_gemm", "moe_gemm_combine", "load_tokens", "add",
                "cross_entropy_tp", "quant_fp8", "gemm_fp8"]
K_GEMM, K_GEMM_RS, K_AG_GEMM, K_RS_ADAMW, K_FSDP_AG_GEMM, K_QUANT_FP8, K_GEMM_FP8 = 5, 20, 21, 22, 23, 30, 31
K_MOE_ROUTE, K_MOE_DISPATCH_GEMM, K_MOE_GEMM_COMBINE = 24, 25, 26
OP_EVENT_RECORD, OP_EVENT_WAIT = 13, 14


class PlanHeader(Structure):
    _fields_ = [("magic", c_uint32), ("version", c_uint32), ("plan_hash", c_uint64), ("topology_hash", c_uint64),
                ("global_rank", c_uint32), ("world_size", c_uint32), ("pipeline_stage", c_uint32),
                ("num_stages", c_uint32), ("tp", c_uint32), ("dp", c_uint32), ("ep", c_uint32), ("cp", c_uint32),
                ("microbatch", c_uint32), ("grad_accum", c_uint32), ("num_microbatches", c_uint32),
                ("seq_len", c_uint32), ("hidden_size", c_uint32), ("layers_in_stage", c_uint32),
                ("num_tensors", c_uint32), ("num_groups", c_uint32), ("num_ops", c_uint32), ("num_events", c_uint32),
                ("arena_bytes", c_uint64), ("global_tokens_per_step", c_uint64), ("flops_per_token_useful", c_uint64),
                ("vpp", c_uint32), ("reserved", c_uint32)]


class TensorDesc(Structure):
    _fields_ = [("offset", c_uint64), ("nbytes", c_uint64), ("shape_id", c_uint32), ("dtype", c_uint16),
                ("tclass", c_uint16)]


class CommGroup(Structure):
    _fields_ = [("group_id", c_uint32), ("kind", c_uint16), ("intra_rack", c_uint16), ("size", c_uint32),
                ("color", c_uint32)]


class Op(Structure):
    _fields_ = [("flops", c_uint64), ("bytes", c_uint64), ("aux0", c_uint32), ("aux1", c_uint32), ("kind", c_uint16),
                ("stream_id", c_uint16), ("exec", c_uint32)]


class Topology(Structure):
    _fields_ = [("gpus_per_rack", c_uint32), ("trays_per_rack", c_uint32), ("gpus_per_tray", c_uint32),
                ("num_racks", c_uint32), ("world_size", c_uint32), ("spare_gpus", c_uint32),
                ("intra_rack_bw", c_uint64), ("inter_rack_bw", c_uint64), ("hbm_bw", c_uint64),
                ("gpu_flops_bf16", c_double), ("gpu_mem_bytes", c_uint64)]


class ModelSpec(Structure):
    _fields_ = [("hidden_size", c_uint32), ("ffn_hidden", c_uint32), ("num_layers", c_uint32), ("num_heads", c_uint32),
                ("num_kv_heads", c_uint32), ("head_dim", c_uint32), ("vocab_size", c_uint32), ("seq_len", c_uint32),
                ("is_moe", c_int32), ("num_experts", c_uint32), ("moe_top_k", c_uint32), ("param_dtype", c_uint16),
                ("optim_dtype", c_uint16), ("optim_states", c_uint32), ("master_weights", c_int32),
                ("recompute", c_int32), ("tp", c_uint32), ("pp", c_uint32), ("ep", c_uint32), ("cp", c_uint32),
                ("vpp", c_uint32), ("microbatch", c_uint32), ("grad_accum", c_uint32), ("mem_budget", c_uint64)]


class TrainSpec(Structure):
    _fields_ = [("lr", c_float), ("beta1", c_float), ("beta2", c_float), ("adam_eps", c_float),
                ("weight_decay", c_float), ("rope_theta", c_float), ("norm_eps", c_float), ("init_std", c_float),
                ("seed", c_uint32), ("tie_embeddings", c_uint32), ("zero_stage", c_uint32), ("fp8_block", c_uint32),
                ("comm_mode", c_uint32), ("ce_chunk", c_uint32), ("moe_capacity_factor_x100", c_uint32),
                ("wgrad_overlap", c_uint32), ("mb_group", c_uint32), ("fuse_swiglu", c_uint32), ("dp_buckets", c_uint32),
                ("wait_limit_ms", c_uint32), ("reserved", c_uint32 * 4)]


class ExecHeader(Structure):
    _fields_ = [("magic", c_uint32), ("num_exec", c_uint32), ("num_named", c_uint32), ("act_slots", c_uint32),
                ("param_elems", c_uint64), ("opt_elems", c_uint64)]


class ExecOp(Structure):
    _fields_ = [("kernel", c_uint16), ("flags", c_uint16), ("t", c_int32 * 8), ("i", c_int32 * 5), ("f", c_float * 2)]


class NamedTensor(Structure):
    _fields_ = [("name", c_char * 40), ("tensor", c_int32), ("grad", c_int32), ("flat_off512", c_int32),
                ("rows", c_uint32), ("cols", c_uint32), ("init_std", c_float)]


assert ctypes.sizeof(PlanHeader) == 128 and ctypes.sizeof(Op) == 32 and ctypes.sizeof(TensorDesc) == 24
assert ctypes.sizeof(Topology) == 64 and ctypes.sizeof(ModelSpec) == 96 and ctypes.sizeof(TrainSpec) == 96
assert ctypes.sizeof(ExecOp) == 64 and ctypes.sizeof(NamedTensor) == 64 and ctypes.sizeof(ExecHeader) == 32


class StepStats(Structure):
    _fields_ = [("step_time_s", c_double), ("busy_compute_s", c_double), ("bubble_ratio", c_double),
                ("mfu", c_double), ("tokens_per_s", c_double), ("tokens_per_s_per_gpu", c_double),
                ("arena_bytes", c_uint64), ("stream_busy", c_double * 6), ("loss", c_double), ("bubble_measured", c_double),
                ("measured", c_uint32), ("reserved", c_uint32)]


class InitDesc(Structure):
    _fields_ = [("global_rank", c_uint32), ("world_size", c_uint32), ("local_rank", c_uint32),
                ("plan_path", c_char_p), ("topology_path", c_char_p), ("checkpoint_path", c_char_p),
                ("checkpoint_every", c_uint32), ("max_steps", c_uint32), ("backend", c_uint32)]


class Batch(Structure):
    _fields_ = [("step", c_uint32), ("tokens", c_uint64), ("seed", c_uint64)]


class PlanError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise PlanError(f"{_LIB_PATH} is missing: run `python -m cai_b200._build` first")
        L = ctypes.CDLL(str(_LIB_PATH))
        L.cai_status_str.restype = c_char_p
        L.cai_log_set_level.argtypes = [c_int]
        L.cai_log_set_level.restype = None
        L.cai_compile.argtypes = [c_char_p, c_char_p, c_uint32, c_uint32, c_uint32, POINTER(c_uint64),
                                  POINTER(c_uint64), c_char_p, c_size_t]
        L.cai_compile_text.argtypes = L.cai_compile.argtypes
        L.cai_verify.argtypes = [c_char_p, c_int, c_char_p, c_size_t]
        L.cai_describe.argtypes = [c_char_p, c_char_p, c_size_t, c_char_p, c_size_t]
        L.cai_group_members.argtypes = [c_char_p, c_uint16, c_uint32, POINTER(c_uint32), c_uint32]
        L.cai_fnv1a64.argtypes = [c_void_p, c_size_t, c_uint64]
        L.cai_fnv1a64.restype = c_uint64
        L.cai_init.argtypes = [POINTER(c_void_p), POINTER(InitDesc)]
        for fn in ("cai_load_plan", "cai_load_checkpoint", "cai_save_checkpoint", "cai_trace_dump_csv", "cai_trace_dump_json"):
            getattr(L, fn).argtypes = [c_void_p, c_char_p]
        L.cai_next_batch.argtypes = [c_void_p, POINTER(Batch)]
        L.cai_train_step.argtypes = [c_void_p, POINTER(Batch)]
        L.cai_should_checkpoint.argtypes = [c_void_p]
        L.cai_last_step_stats.argtypes = [c_void_p, POINTER(StepStats)]
        L.cai_trace_enable.argtypes = [c_void_p, c_int]
        L.cai_finalize.argtypes = [c_void_p]
        L.cai_current_step.argtypes = [c_void_p]
        L.cai_current_step.restype = c_uint32
        L.cai_ckpt_write.argtypes = [c_char_p, c_char_p, c_uint32, c_uint32, c_uint64, c_uint32, POINTER(c_char_p),
                                     POINTER(c_void_p), POINTER(c_uint64)]
        L.cai_ckpt_write2.argtypes = [c_char_p, c_char_p, c_uint32, c_uint32, c_uint64, c_uint32, POINTER(c_char_p),
                                      POINTER(c_void_p), POINTER(c_uint64), c_int]
        L.cai_ckpt_probe.argtypes = [c_char_p, c_uint32, POINTER(c_uint32), POINTER(c_uint64), POINTER(c_uint32),
                                     c_char_p, c_size_t]
        L.cai_ckpt_section.argtypes = [c_char_p, c_uint32, c_char_p, POINTER(c_uint64), c_void_p, c_uint64]
        _lib = L
    return _lib


def fnv1a(data: bytes, seed: int = 0) -> int:
    return lib().cai_fnv1a64(data, len(data), seed)


class PipelineStats(ctypes.Structure):
    _fields_ = [("n_stages", c_uint32), ("reserved", c_uint32), ("step_time_s", c_double), ("bubble_formula", c_double),
                ("bubble_replayed", c_double), ("tokens_per_s", c_double), ("mfu", c_double),
                ("stage_finish_s", c_double * 64), ("stage_busy_hi_s", c_double * 64), ("stage_idle_hi", c_double * 64),
                ("stage_sm_busy_s", c_double * 64)]


def pipeline_replay(plan_paths, topology_path, backend="calibrated", calibration=None, trace=None) -> dict:
    """Replay the plans of all stages of one pipeline together (``plan_paths[s]``: one rank of stage ``s``): sends meet
    their receives, so fill, drain, uneven stages and transfer times are in the step time without the closed bubble
    formula the single-plan replay (and the reference, src/runtime.c:191-194) applies. ``trace``: path of a Trace
    Event JSON timeline with one process per stage. Raises ``PlanError`` when the stages' sends and receives deadlock."""
    paths = [str(p).encode() for p in plan_paths]
    arr = (c_char_p * len(paths))(*paths)
    st = PipelineStats()
    err = ctypes.create_string_buffer(512)
    L = lib()
    L.cai_pipeline_replay.argtypes = [POINTER(c_char_p), c_uint32, c_char_p, c_uint32, c_char_p, c_char_p, POINTER(PipelineStats),
                                      c_char_p, c_size_t]
    rc = L.cai_pipeline_replay(arr, len(paths), str(topology_path).encode(), BACKENDS[backend],
                               str(calibration).encode() if calibration else None, str(trace).encode() if trace else None,
                               ctypes.byref(st), err, len(err))
    if rc != 0:
        raise PlanError(f"pipeline replay failed ({L.cai_status_str(rc).decode()}): {err.value.decode()}")
    n = st.n_stages
    return {"step_time_s": st.step_time_s, "bubble_formula": st.bubble_formula, "bubble_replayed": st.bubble_replayed,
            "tokens_per_s": st.tokens_per_s, "mfu": st.mfu, "stage_finish_s": list(st.stage_finish_s[:n]),
            "stage_busy_hi_s": list(st.stage_busy_hi_s[:n]), "stage_idle_hi": list(st.stage_idle_hi[:n]),
            "stage_sm_busy_s": list(st.stage_sm_busy_s[:n])}


LOG_LEVELS = {"error": 0, "warn": 1, "info": 2, "debug": 3}


def set_log_level(level) -> None:
    """Level of the native library's stderr log (``"error" | "warn" | "info" | "debug"`` or 0..3); the environment
    variable CAI_LOG_LEVEL sets the starting level of a process (default info, as in the reference, src/common.c:9-22)."""
    lib().cai_log_set_level(LOG_LEVELS[level] if isinstance(level, str) else int(level))


def compile_plans(config, outdir, ranks=None, version=2, text=False):
    """Compile ``config`` (a path, or config text with ``text=True``) into ``outdir``.

    ``ranks`` is ``(lo, hi)``; default is every rank. Returns ``(plan_hash, topology_hash)``.
    """
    ph, th = c_uint64(0), c_uint64(0)
    err = ctypes.create_string_buffer(512)
    lo, hi = ranks if ranks is not None else (0, 0xFFFFFFFF)
    fn = lib().cai_compile_text if text else lib().cai_compile
    rc = fn(str(config).encode(), str(outdir).encode() if outdir else None, lo, hi, version, ctypes.byref(ph),
            ctypes.byref(th), err, len(err))
    if rc != 0:
        raise PlanError(f"compile failed ({lib().cai_status_str(rc).decode()}): {err.value.decode()}")
    return ph.value, th.value


def describe(config_text: str) -> dict:
    out = ctypes.create_string_buffer(8192)
    err = ctypes.create_string_buffer(512)
    rc = lib().cai_describe(config_text.encode(), out, len(out), err, len(err))
    if rc != 0:
        raise PlanError(f"describe failed: {err.value.decode()}")
    d = {}
    for line in out.value.decode().splitlines():
        k, _, v = line.partition("=")
        try:
            d[k] = int(v)
        except ValueError:
            try:
                d[k] = float(v)
            except ValueError:
                d[k] = v
    return d


def group_members(config_text: str, kind: int, rank: int):
    buf = (c_uint32 * 65536)()
    n = lib().cai_group_members(config_text.encode(), kind, rank, buf, len(buf))
    if n < 0:
        raise PlanError("group_members failed")
    return [buf[i] for i in range(n)]


def verify(config_path, check_exec=True):
    """Whole-cluster verification. Returns ``(problems, report_text)``."""
    buf = ctypes.create_string_buffer(1 << 20)
    rc = lib().cai_verify(str(config_path).encode(), int(check_exec), buf, len(buf))
    return rc, buf.value.decode()


def lint(config_path):
    """Pre-compile checks of a configuration (what ``bin/topology_linter`` prints). Returns ``(failed, report_text)``."""
    buf = ctypes.create_string_buffer(1 << 16)
    rc = lib().cai_lint(str(config_path).encode(), buf, len(buf))
    return rc, buf.value.decode()


TENSOR_CLASSES = ("param", "grad", "optstate", "activation", "comm", "workspace")


class PlanFile:
    """A plan file parsed into ctypes arrays (version 1 or 2)."""

    def class_bytes(self) -> dict:
        """Bytes every tensor class occupies in the arena (extent of the class's tensors; same rule as the C++
        ``plan_class_bytes``): what a device allocates, as opposed to the memory model of the decomposition report."""
        lo = [None] * len(TENSOR_CLASSES)
        hi = [0] * len(TENSOR_CLASSES)
        for t in self.tensors:
            if t.tclass >= len(TENSOR_CLASSES) or t.nbytes == 0:
                continue
            lo[t.tclass] = t.offset if lo[t.tclass] is None else min(lo[t.tclass], t.offset)
            hi[t.tclass] = max(hi[t.tclass], t.offset + t.nbytes)
        return {n: (hi[i] - lo[i] if lo[i] is not None else 0) for i, n in enumerate(TENSOR_CLASSES)}

    def __init__(self, path):
        self.path = str(path)
        self.raw = Path(path).read_bytes()
        off = 0

        def take(ctype, count=1):
            nonlocal off
            size = ctypes.sizeof(ctype) * count
            if off + size > len(self.raw):
                raise PlanError(f"{path}: truncated plan file")
            arr = (ctype * count).from_buffer_copy(self.raw, off)
            off += size
            return arr

        self.hdr = take(PlanHeader)[0]
        if self.hdr.magic != PLAN_MAGIC or self.hdr.version not in (1, 2):
            raise PlanError(f"{path}: not a plan file")
        self.tensors = take(TensorDesc, self.hdr.num_tensors)
        self.groups = take(CommGroup, self.hdr.num_groups)
        self.ops = take(Op, self.hdr.num_ops)
        self.exec = self.named = self.shapes = None
        self.train = self.model = self.xhdr = None
        if self.hdr.version >= 2:
            self.xhdr = take(ExecHeader)[0]
            if self.xhdr.magic != EXEC_MAGIC:
                raise PlanError(f"{path}: bad execution section")
            self.train = take(TrainSpec)[0]
            self.model = take(ModelSpec)[0]
            self.exec = take(ExecOp, self.xhdr.num_exec)
            self.named = take(NamedTensor, self.xhdr.num_named)
            self.shapes = take(c_uint32, self.hdr.num_tensors * 4)

    def named_dict(self):
        return {n.name.decode(): n for n in self.named}

    def shape(self, tensor):
        return self.shapes[tensor * 4], self.shapes[tensor * 4 + 1], self.shapes[tensor * 4 + 2]


def read_topology(path) -> Topology:
    raw = Path(path).read_bytes()
    if len(raw) != 68 or int.from_bytes(raw[:4], "little") != TOPO_MAGIC:
        raise PlanError(f"{path}: not a topology file")
    return Topology.from_buffer_copy(raw, 4)


BACKENDS = {"default": 0, "analytic": 1, "device": 2, "auto": 3, "calibrated": 4}


class Simulator:
    """Replay of a plan through the C API (the reference's ``trainer`` behaviour). ``backend``: "analytic" prices ops
    from FLOPs and bytes over the datasheet figures (the reference's model), "calibrated" prices version-2 plans with
    costs fitted to this repository's kernels as measured on B200s (``calibration``: optional key = value file that
    overrides constants), "device" / "auto" execute on a GPU."""

    def __init__(self, plan_path, topology_path, rank=0, checkpoint_path=None, checkpoint_every=0, max_steps=0,
                 backend="default", calibration=None):
        self._keep = [str(plan_path).encode(), str(topology_path).encode(),
                      str(checkpoint_path).encode() if checkpoint_path else None]
        if calibration is not None:
            os.environ["CAI_CALIBRATION"] = str(calibration)
        elif backend == "calibrated":
            os.environ.pop("CAI_CALIBRATION", None)
        d = InitDesc(rank, 0, 0, self._keep[0], self._keep[1], self._keep[2], checkpoint_every, max_steps, BACKENDS[backend])
        self.ctx = c_void_p()
        rc = lib().cai_init(ctypes.byref(self.ctx), ctypes.byref(d))
        if rc != 0:
            raise PlanError(f"cai_init failed: {lib().cai_status_str(rc).decode()}")

    def load_checkpoint(self, path):
        return lib().cai_load_checkpoint(self.ctx, str(path).encode())

    def step(self):
        b = Batch()
        if lib().cai_next_batch(self.ctx, ctypes.byref(b)) != 0:
            return None
        rc = lib().cai_train_step(self.ctx, ctypes.byref(b))
        if rc != 0:
            raise PlanError(f"train_step failed: {lib().cai_status_str(rc).decode()}")
        s = StepStats()
        lib().cai_last_step_stats(self.ctx, ctypes.byref(s))
        return s

    @property
    def current_step(self):
        return lib().cai_current_step(self.ctx)

    def should_checkpoint(self):
        return bool(lib().cai_should_checkpoint(self.ctx))

    def save_checkpoint(self, tag):
        return lib().cai_save_checkpoint(self.ctx, tag.encode())

    def trace(self, on=True):
        lib().cai_trace_enable(self.ctx, int(on))

    def dump_trace(self, path):
        """CSV in the reference's schema, or (path ending in .json) the Trace Event format of chrome://tracing / Perfetto."""
        fn = lib().cai_trace_dump_json if str(path).endswith(".json") else lib().cai_trace_dump_csv
        return fn(self.ctx, str(path).encode())

    def close(self):
        if self.ctx:
            lib().cai_finalize(self.ctx)
            self.ctx = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
