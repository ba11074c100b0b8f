"""A reference interpreter of executable plans on the CPU: a test oracle for the schedule, not a backend.

The plan compiler turns a configuration into one op table per rank: kernel records over tensors of a static arena, in
issue order over six streams, with the collectives and the pipeline hand-offs of the layout. The GPU executor runs those
tables with the sm_100a kernels; this module runs the same tables with plain PyTorch arithmetic on the host, every rank
of the job inside one process, so that what a layout computes can be checked without a GPU: a job of tp x pp x dp ranks
must train exactly like the one-device model (``reference_torch.forward_loss`` + AdamW), because every collective,
every hand-off and every shard boundary in the tables is executed for real.

What is interpreted: the decoder under tensor (fused or NCCL-only plans), pipeline and data parallelism with
sharded optimizer state (the fused reduce-scatter + AdamW kernel in its whole-space and its per-layer bucket form) or
with parameters and gradients sharded too (ZeRO-3: parameter gathers, staged gradients, owners' accumulators). Each record does what the kernel it names is specified to do (``csrc/kernels/cai_kernels.h``,
``csrc/comm/fused.h``): tensors keep their storage types (bf16 activations and weights, fp32 gradients and optimizer
state, e4m3 operands with their block scales under ``param_dtype = fp8e4m3``), arithmetic inside a record is fp32.
Mixture-of-experts plans are interpreted too: router, slot assignment in token order, dispatch into the owners' slabs,
the experts' products over the live rows of the slabs, combine, and the backward of all of it. A record without an
interpretation raises ``NotImplementedError``.

By default every rank issues its table in program order. That order is a legal serialisation of a rank's streams (a
wait never precedes its record in a table); a collective runs when every member of its group has reached it; a
pipeline send deposits its message and continues, a receive blocks until the message is there. A job whose ranks
cannot all finish raises instead of hanging. With ``order = "random"`` the six streams of every rank advance
independently, held back only by the plan's own record / wait events, and the next op is drawn at random among all that
may start: a dynamic check that the events order every dependence (the static proof is ``verify_hazards``).
"""
from __future__ import annotations

import random
import tempfile
from collections import defaultdict, deque
from pathlib import Path

import numpy as np
import torch

from .. import plan as planlib
from ..utils import reshard

K = {name: i for i, name in enumerate(planlib.KERNEL_NAMES)}
_TORCH = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16, 3: torch.float8_e4m3fn, 5: torch.int32, 6: torch.uint8}
ST_IO = 5


class _Rank:
    def __init__(self, pf: planlib.PlanFile, rank: int):
        self.pf, self.rank = pf, rank
        self.rl = reshard.RankLayout(pf, rank)
        self.arena = torch.zeros(int(pf.hdr.arena_bytes) + 16, dtype=torch.uint8)
        self.named = pf.named_dict()
        self._typed = {}

    def _base(self, dtype):
        if dtype not in self._typed:
            n = self.arena.numel() // torch.empty(0, dtype=dtype).element_size() * torch.empty(0, dtype=dtype).element_size()
            self._typed[dtype] = self.arena[:n].view(dtype)
        return self._typed[dtype]

    def mat(self, tid, rows=None, cols=None):
        """Pitched 2-D view of a tensor; ``rows`` / ``cols`` override the table's extent (a record names its own)."""
        t = self.pf.tensors[tid]
        r, c, ld = self.pf.shape(tid)
        dt = _TORCH[t.dtype]
        es = planlib.DTYPE_SIZE[t.dtype]
        rows, cols = r if rows is None else rows, c if cols is None else cols
        ld = ld or cols
        need = ((rows - 1) * ld + cols) * es if rows and cols else 0
        if need > t.nbytes:
            raise ValueError(f"tensor {tid}: a record addresses {need} bytes of {t.nbytes}")
        return torch.as_strided(self._base(dt), (rows, cols), (ld, 1), t.offset // es)

    def flat(self, tid, count=None):
        t = self.pf.tensors[tid]
        es = planlib.DTYPE_SIZE[t.dtype]
        n = t.nbytes // es if count is None else count
        if n * es > t.nbytes:
            raise ValueError(f"tensor {tid}: a record addresses {n * es} bytes of {t.nbytes}")
        return self._base(_TORCH[t.dtype])[t.offset // es:t.offset // es + n]

    def named_flat(self, name):
        return self.flat(self.named[name].tensor)


def _rope(x, seq, theta, inverse):
    """x [T, heads, hd] fp32, position of row t is t % seq; rotate-half convention (``reference_torch.rope``)."""
    T, _, hd = x.shape
    half = hd // 2
    pos = (torch.arange(T) % seq).to(torch.float32)
    inv = theta ** (-torch.arange(half, dtype=torch.float32) / half)
    ang = pos[:, None] * inv[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    if inverse:
        s = -s
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


def _attention(q, k, v, B, S, scale):
    """q [B*S, nh, hd], k / v [B*S, nkv, hd] fp32 -> out [B*S, nh*hd], causal, grouped-query."""
    nh, nkv, hd = q.shape[1], k.shape[1], q.shape[2]
    qh = q.view(B, S, nh, hd).transpose(1, 2)
    kh = k.view(B, S, nkv, hd).transpose(1, 2).repeat_interleave(nh // nkv, 1)
    vh = v.view(B, S, nkv, hd).transpose(1, 2).repeat_interleave(nh // nkv, 1)
    s = (qh @ kh.transpose(-1, -2)) * scale
    s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
    lse = torch.logsumexp(s, -1)                                   # [B, nh, S]
    out = torch.softmax(s, -1) @ vh
    return out.transpose(1, 2).reshape(B * S, nh * hd), lse


class PlanInterpreter:
    """All ranks of one job, interpreted on the host. ``config_text``: the job's configuration (executable layout)."""

    def __init__(self, config_text: str, order: str = "program", seed: int = 0):
        if order not in ("program", "random"):
            raise ValueError("order is 'program' or 'random'")
        self.order, self.seed = order, seed
        self.config_text = config_text
        d = planlib.describe(config_text)
        self.world = int(d["world_size"])
        with tempfile.TemporaryDirectory(prefix="cai_interp_") as tmp:
            planlib.compile_plans(config_text, tmp, ranks=(0, self.world), version=2, text=True)
            self.ranks = [_Rank(planlib.PlanFile(Path(tmp) / f"plan.rank{r:06d}.bin"), r) for r in range(self.world)]
        pf = self.ranks[0].pf
        self.train, self.model, self.hdr = pf.train, pf.model, pf.hdr
        self.step_count = 0
        self.lr = float(self.train.lr)
        self._members = {}
        self.rows_per_replica = int(self.hdr.num_microbatches * self.hdr.microbatch)

    # ------------------------------------------------------------------ state in, state out
    def layouts(self):
        return [r.rl for r in self.ranks]

    def load_state(self, state, step=0):
        """``state[name][key]``: global fp32 ``master`` / ``m`` / ``v`` tensor of every parameter (the form
        ``cai_b200.utils.reshard`` works on). Every rank receives what a checkpoint of its layout would hold."""
        for r in self.ranks:
            sec = reshard.rank_sections(r.rl, state, step)
            for key, name in (("master", "@flat_master"), ("m", "@flat_m"), ("v", "@flat_v")):
                dst = r.named_flat(name)
                dst[:len(sec[key])].copy_(torch.from_numpy(sec[key]))
            p = r.named_flat("@flat_param")
            p[:len(sec["param"])].copy_(torch.from_numpy(sec["param"]).view(torch.bfloat16))
        self.step_count = step

    def state(self):
        """The global state back out of the ranks' buffers (same form as ``load_state`` takes)."""
        def read(rank):
            r = self.ranks[rank]
            out = {"plan_hash": r.rl.plan_hash, "step": self.step_count}
            for key, name in (("master", "@flat_master"), ("m", "@flat_m"), ("v", "@flat_v")):
                out[key] = r.named_flat(name).numpy().copy()
            return out
        return reshard.gather_global(self.layouts(), read)[0]

    def parameter(self, rank, name):
        """One rank's bf16 shard of a parameter as fp32 (what its kernels read)."""
        r = self.ranks[rank]
        nt = r.named[name]
        return r.mat(nt.tensor).float()

    # ------------------------------------------------------------------ one optimizer step
    def step(self, tokens, targets, lr=None) -> float:
        """``tokens`` / ``targets``: int tensors ``[global sequences, seq]``; data-parallel replica ``d`` takes rows
        ``[d * rows, (d + 1) * rows)``. Returns the mean loss over the global batch."""
        self.step_count += 1
        t = self.step_count
        b1, b2 = float(self.train.beta1), float(self.train.beta2)
        self.hyper = (float(self.lr if lr is None else lr), b1, b2, float(self.train.adam_eps), float(self.train.weight_decay),
                      1.0 - b1 ** t, 1.0 - b2 ** t)
        rows = self.rows_per_replica
        if tokens.shape[0] != rows * int(self.hdr.dp) or tokens.shape != targets.shape or tokens.shape[1] != int(self.model.seq_len):
            raise ValueError(f"a step of this job takes {rows * int(self.hdr.dp)} sequences of {int(self.model.seq_len)} tokens, "
                             f"got {tuple(tokens.shape)}")
        for r in self.ranks:
            d = r.rl.dp_id
            for name, src in (("@tokens", tokens), ("@targets", targets)):
                dst = r.named_flat(name)
                part = src[d * rows:(d + 1) * rows].reshape(-1).to(torch.int32)
                dst[:part.numel()].copy_(part)
        self._run()
        # the last stage accumulates the loss; the plan all-reduces it over the tensor- and data-parallel groups
        last = next(r for r in self.ranks if r.rl.stage == r.rl.pp - 1)
        return float(last.named_flat("@loss")[0].item())

    # ------------------------------------------------------------------ scheduler
    def members(self, kind, rank):
        key = (kind, rank)
        if key not in self._members:
            self._members[key] = planlib.group_members(self.config_text, kind, rank)
        return self._members[key]

    def expert_group(self, r):
        """Members of the group the experts are spread over, in member order: the tp ranks of each of the ep replicas
        of the rank's block (member = replica * tp + tp rank), as ``cai_b200.parallel.peers`` maps them on the device."""
        h = self.hdr
        tp, ep = int(h.tp), max(1, int(h.ep))
        replica = tp * int(h.num_stages) * max(1, int(h.cp))
        tp_id, within, dp_id = r.rank % tp, r.rank % replica, r.rank // replica
        first_dp = (dp_id // ep) * ep
        return [within - tp_id + t + (first_dp + i) * replica for i in range(ep) for t in range(tp)]

    def _run(self):
        """One optimizer step of every rank. ``order = "program"``: each rank issues its table in program order (one
        legal serialisation of its streams). ``order = "random"``: every rank keeps one queue per stream, a record marks
        its event when the stream reaches it, a wait holds its stream until the event is marked, and among all ops that
        could start the next one is drawn at random: any interleaving the events of the plan allow. A plan whose events
        order every dependence gives the same result under every such interleaving; a missing edge shows as a result
        that depends on the draw."""
        self.mail = defaultdict(deque)          # (src rank, dst rank, channel) -> messages
        self.pending = {}                       # collective key -> {rank: request}
        self.calls = defaultdict(int)           # per rank and channel: collectives issued so far
        rng = random.Random(self.seed * 1000003 + self.step_count)
        queues, recorded_before, marked = {}, {}, {}
        for r in self.ranks:
            ops = r.pf.ops
            marked[r.rank] = set()
            if self.order == "program":
                queues[(r.rank, 0)] = deque(i for i, op in enumerate(ops)
                                            if op.exec and op.kind not in (planlib.OP_EVENT_RECORD, planlib.OP_EVENT_WAIT))
                continue
            seen = set()
            for i, op in enumerate(ops):
                if op.kind == planlib.OP_EVENT_WAIT:
                    recorded_before[(r.rank, i)] = op.aux0 in seen      # a wait on an event nothing recorded yet passes at once
                elif op.kind == planlib.OP_EVENT_RECORD:
                    seen.add(op.aux0)
                elif not op.exec:
                    continue
                queues.setdefault((r.rank, int(op.stream_id)), deque()).append(i)
        waiting = {}                            # queue -> what its head op waits for
        while True:
            live = [key for key, dq in queues.items() if dq]
            if not live:
                return
            runnable = []
            for key in live:
                rank, i = key[0], queues[key][0]
                if key in waiting:
                    if self._ready(waiting[key]):
                        runnable.append(key)
                    continue
                op = self.ranks[rank].pf.ops[i]
                if op.kind == planlib.OP_EVENT_WAIT and recorded_before[(rank, i)] and op.aux0 not in marked[rank]:
                    continue
                runnable.append(key)
            if not runnable:
                stuck = {key: waiting.get(key, "an event") for key in live}
                raise RuntimeError(f"the ranks wait for each other and none can continue: {stuck}")
            # program order: stay with the lowest rank until it blocks (deterministic); random: any op that may start
            key = runnable[0] if self.order == "program" else rng.choice(runnable)
            r = self.ranks[key[0]]
            i = queues[key][0]
            op = r.pf.ops[i]
            if op.kind == planlib.OP_EVENT_RECORD:
                marked[r.rank].add(op.aux0)
                queues[key].popleft()
                continue
            if op.kind == planlib.OP_EVENT_WAIT:
                queues[key].popleft()
                continue
            token = self._issue(r, op, resumed=waiting.pop(key, None))
            if token is None:
                queues[key].popleft()
            else:
                waiting[key] = token

    def _ready(self, want):
        what = want[0]
        if what == "recv":
            return bool(self.mail[want[1]])
        if what == "coll":
            return want[1] not in self.pending      # the last member to arrive ran it and removed the entry
        return True

    def _collective(self, r, key, members, fn, payload):
        """Join one collective call; the last member to arrive runs ``fn`` for the whole group."""
        slot = self.pending.setdefault(key, {})
        slot[r.rank] = payload
        if len(slot) == len(members):
            fn([self.ranks[m] for m in members], [slot[m] for m in members])
            del self.pending[key]
            return None
        return ("coll", key)

    # ------------------------------------------------------------------ one op of a rank
    def _issue(self, r: _Rank, op, resumed=None):
        """Runs the op, or returns what it has to wait for (``resumed``: the wait it came back from)."""
        x = r.pf.exec[op.exec - 1]
        k = int(x.kernel)
        if resumed is not None and resumed[0] == "coll":
            return None                                         # the last member to arrive ran it for everyone
        handler = self._local.get(k)
        if handler is not None:
            handler(self, r, x)
            return None
        if k == K["nccl_send"]:
            peer = self.members(planlib.GROUP_PP, r.rank)[x.i[4]]
            self.mail[(r.rank, peer, int(op.stream_id == ST_IO))].append(r.flat(x.t[0], self._count(x)).clone())
            return None
        if k == K["nccl_recv"]:
            peer = self.members(planlib.GROUP_PP, r.rank)[x.i[4]]
            key = (peer, r.rank, int(op.stream_id == ST_IO))
            if not self.mail[key]:
                return ("recv", key)
            r.flat(x.t[1], self._count(x)).copy_(self.mail[key].popleft())
            return None
        coll = self._group_ops.get(k)
        if coll is None:
            raise NotImplementedError(f"kernel '{planlib.KERNEL_NAMES[k]}' is not interpreted")
        if k in (K["moe_dispatch_gemm"], K["moe_gemm_combine"]):
            members = tuple(self.expert_group(r))
        else:
            kind = (planlib.GROUP_TP if k == K["cross_entropy_tp"] else planlib.GROUP_DP if k == K["fsdp_ag_gemm"] else int(x.i[3]))
            members = tuple(self.members(kind, r.rank))
        # which call of the group this is: the fused kernels carry a sequence number (their signal epoch); NCCL calls of
        # one communicator match in issue order, and a communicator belongs to one stream (the vocabulary-parallel
        # cross-entropy has the tensor-parallel group's second one)
        if k in (K["nccl_all_reduce"], K["nccl_reduce_scatter"], K["nccl_all_gather"], K["cross_entropy_tp"]):
            lane = ("ce",) if k == K["cross_entropy_tp"] else ("nccl", int(op.stream_id))
            n = self.calls[(r.rank, members, lane)]
            self.calls[(r.rank, members, lane)] += 1
            key = (members, lane, n)
        else:
            key = (members, "seq", int(x.i[4]), self.step_count)
        return self._collective(r, key, members, coll.__get__(self), x)

    # ------------------------------------------------------------------ records of one rank
    def _gemm_core(self, r, A, B, M, N, Kd, ta, tb):
        a = r.mat(A, Kd if ta else M, M if ta else Kd).float()
        b = r.mat(B, Kd if tb else N, N if tb else Kd).float()
        return (a.t() if ta else a) @ (b if tb else b.t())

    def _epilogue(self, r, acc, x, C, R, epi, alpha=1.0):
        M, N = acc.shape
        acc = acc * alpha
        if epi == 0:
            r.mat(C, M, N).copy_(acc)
        elif epi == 1:
            r.mat(C, M, N).copy_(acc)
        elif epi == 2:
            c = r.mat(C, M, N)
            c.copy_(c + acc)
        elif epi == 3:
            r.mat(C, M, N).copy_(acc + r.mat(R, M, N).float())
        elif epi == 4:      # SwiGLU forward: C = [gate | up], R (an output) = silu(gate) * up
            F = N // 2
            r.mat(C, M, N).copy_(acc)
            g, u = acc[:, :F], acc[:, F:]
            r.mat(R, M, F).copy_(g * torch.sigmoid(g) * u)
        elif epi == 5:      # SwiGLU backward: acc = dact [M, F]; R = saved [gate | up]; C = [dgate | dup]
            F = N
            gu = r.mat(R, M, 2 * F).float()
            g, u = gu[:, :F], gu[:, F:]
            sg = torch.sigmoid(g)
            r.mat(C, M, 2 * F).copy_(torch.cat([acc * u * sg * (1 + g * (1 - sg)), acc * g * sg], 1))
        else:
            raise NotImplementedError(f"GEMM epilogue {epi}")

    def _k_gemm_slabs(self, r, x):
        """The products of the local experts over their ragged slabs. Group g reads A, B at row g * (rows of one group)
        and writes C likewise; the segmented dimension is cut into sub-slabs of ``seg_rows`` rows of which only the first
        ``counts[...]`` hold data: mode 1 segments M (rows past a count are not written), mode 2 segments K (rows past a
        count do not contribute: the weight gradient)."""
        ta, tb, epi = x.flags & 1, (x.flags >> 1) & 1, (x.flags >> 4) & 0xF
        M, N, Kd, seg_rows = x.i[0], x.i[1], x.i[2], x.i[3]
        seg_mode, groups = x.i[4] & 0xFF, (x.i[4] >> 8) if x.flags & 0x100 else 1
        ga, gb = (Kd if ta else M), (Kd if tb else N)
        a_all = r.mat(x.t[0], groups * ga, M if ta else Kd).float()
        b_all = r.mat(x.t[1], groups * gb, N if tb else Kd).float()
        c_all = r.mat(x.t[2], groups * M, N)
        per = (Kd if seg_mode == 2 else M) // seg_rows
        counts = r.flat(x.t[4], groups * per).long()
        for g in range(groups):
            a, b = a_all[g * ga:(g + 1) * ga], b_all[g * gb:(g + 1) * gb]
            a, b = (a.t() if ta else a), (b if tb else b.t())            # [M, K], [K, N]
            live = torch.zeros(per * seg_rows, dtype=torch.bool)
            for j in range(per):
                live[j * seg_rows:j * seg_rows + int(counts[g * per + j])] = True
            c = c_all[g * M:(g + 1) * M]
            if seg_mode == 2:
                acc = (a[:, live] @ b[live]) * float(x.f[0])
                c.copy_(c + acc if epi == 2 else acc)
            else:
                acc = (a[live] @ b) * float(x.f[0])
                c[live] = (c[live].float() + acc if epi == 2 else acc).to(c.dtype)

    def _k_gemm(self, r, x):
        if x.flags & 0x100 or x.t[4] >= 0:
            return self._k_gemm_slabs(r, x)
        ta, tb, epi = x.flags & 1, (x.flags >> 1) & 1, (x.flags >> 4) & 0xF
        acc = self._gemm_core(r, x.t[0], x.t[1], x.i[0], x.i[1], x.i[2], ta, tb)
        self._epilogue(r, acc, x, x.t[2], x.t[3], epi, float(x.f[0]))

    @staticmethod
    def _quant(v, rows_per_scale, cols_per_scale=128):
        """e4m3 with one scale (amax / 448) per ``rows_per_scale x cols_per_scale`` block; returns (q as fp32 values, scale)."""
        R, C = v.shape
        br, bc = -(-R // rows_per_scale), -(-C // cols_per_scale)
        pad = torch.zeros(br * rows_per_scale, bc * cols_per_scale)
        pad[:R, :C] = v
        blocks = pad.view(br, rows_per_scale, bc, cols_per_scale)
        scale = blocks.abs().amax((1, 3)) / 448.0
        safe = torch.where(scale > 0, scale, torch.ones_like(scale))
        q = (blocks / safe[:, None, :, None]).to(torch.float8_e4m3fn).float().view(br * rows_per_scale, bc * cols_per_scale)[:R, :C]
        return q, scale

    def _k_quant_fp8(self, r, x):
        rows, cols = x.i[0], x.i[1]
        v = r.mat(x.t[0], rows, cols).float()
        if x.flags & 1:     # a weight: 128 x 128 blocks, and the transposed copy with its own scale table
            q, sc = self._quant(v, 128)
            r.mat(x.t[1], rows, cols).copy_(q)
            r.mat(x.t[2], -(-rows // 128), -(-cols // 128)).copy_(sc)
            if x.t[3] >= 0:
                r.mat(x.t[3], cols, rows).copy_(q.t())
                r.mat(x.t[4], -(-cols // 128), -(-rows // 128)).copy_(sc.t())
        else:               # an activation: one scale per row and 128 columns
            q, sc = self._quant(v, 1)
            r.mat(x.t[1], rows, cols).copy_(q)
            r.mat(x.t[2], rows, cols // 128).copy_(sc)

    def _k_gemm_fp8(self, r, x):
        """C[M,N] = sum over 128-wide k blocks of sa[m,kb] * sb[n/128,kb] * (Aq[m,kb] . Bq[n,kb])."""
        M, N, Kd = x.i[0], x.i[1], x.i[2]
        a = r.mat(x.t[0], M, Kd).float() * r.mat(x.t[4], M, Kd // 128).float().repeat_interleave(128, 1)
        sb = r.mat(x.t[5], -(-N // 128), Kd // 128).float().repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)
        b = r.mat(x.t[1], N, Kd).float() * sb
        self._epilogue(r, a @ b.t(), x, x.t[2], x.t[3], (x.flags >> 4) & 0xF)

    def _k_embed_fwd(self, r, x):
        T, H, lo, hi = x.i[0], x.i[1], x.i[2], x.i[3]
        tok = r.flat(x.t[0], T).long()
        E = r.mat(x.t[1], hi - lo, H)
        own = (tok >= lo) & (tok < hi)
        out = torch.zeros(T, H)
        out[own] = E[tok[own] - lo].float()
        r.mat(x.t[2], T, H).copy_(out)

    def _k_embed_bwd(self, r, x):
        T, H, lo, hi = x.i[0], x.i[1], x.i[2], x.i[3]
        tok = r.flat(x.t[0], T).long()
        own = (tok >= lo) & (tok < hi)
        dE = r.mat(x.t[2], hi - lo, H)
        dE.index_add_(0, tok[own] - lo, r.mat(x.t[1], T, H).float()[own])

    def _k_rmsnorm_fwd(self, r, x):
        rows, H = x.i[0], x.i[1]
        v = r.mat(x.t[0], rows, H).float()
        rstd = torch.rsqrt(v.pow(2).mean(-1) + float(x.f[0]))
        r.mat(x.t[2], rows, H).copy_(v * rstd[:, None] * r.flat(x.t[1], H).float())
        r.flat(x.t[3], rows).copy_(rstd)

    def _k_rmsnorm_bwd(self, r, x):
        rows, H, dx_acc, dg_acc = x.i[0], x.i[1], x.i[2], x.i[3]
        v, g = r.mat(x.t[0], rows, H).float(), r.flat(x.t[1], H).float()
        rstd, dy = r.flat(x.t[2], rows).float(), r.mat(x.t[3], rows, H).float()
        xhat = v * rstd[:, None]
        dyg = dy * g
        dx = rstd[:, None] * (dyg - xhat * (dyg * xhat).mean(-1, keepdim=True))
        dst = r.mat(x.t[4], rows, H)
        dst.copy_(dst.float() + dx if dx_acc else dx)
        dg = r.flat(x.t[5], H)
        part = (dy * xhat).sum(0)
        dg.copy_(dg + part if dg_acc else part)

    def _k_rope(self, r, x):
        T, seq, nh, nkv, hd = x.i[0], x.i[1], x.i[2], x.i[3], x.i[4]
        qkv = r.mat(x.t[0], T, (nh + 2 * nkv) * hd)
        qk = qkv[:, :(nh + nkv) * hd].float().view(T, nh + nkv, hd)
        qkv[:, :(nh + nkv) * hd].copy_(_rope(qk, seq, float(self.train.rope_theta), bool(x.flags & 1)).reshape(T, -1))

    def _split_qkv(self, r, tid, T, nh, nkv, hd):
        qkv = r.mat(tid, T, (nh + 2 * nkv) * hd).float()
        q, kk, v = qkv.split([nh * hd, nkv * hd, nkv * hd], 1)
        return q.reshape(T, nh, hd), kk.reshape(T, nkv, hd), v.reshape(T, nkv, hd)

    def _k_attn_fwd(self, r, x):
        B, S, nh, nkv, hd = x.i[0], x.i[1], x.i[2], x.i[3], x.i[4]
        q, kk, v = self._split_qkv(r, x.t[0], B * S, nh, nkv, hd)
        out, lse = _attention(q, kk, v, B, S, float(x.f[0]))
        r.mat(x.t[1], B * S, nh * hd).copy_(out)
        r.flat(x.t[2], B * nh * S).copy_(lse.reshape(-1))

    def _k_attn_bwd(self, r, x):
        parts = int(x.flags) or 7
        if not parts & 6:
            return              # the row sums alone: an intermediate of the kernels, not needed here
        B, S, nh, nkv, hd = x.i[0], x.i[1], x.i[2], x.i[3], x.i[4]
        T = B * S
        q, kk, v = (t.clone().requires_grad_(True) for t in self._split_qkv(r, x.t[0], T, nh, nkv, hd))
        out, _ = _attention(q, kk, v, B, S, float(x.f[0]))
        out.backward(r.mat(x.t[2], T, nh * hd).float())
        dqkv = r.mat(x.t[5], T, (nh + 2 * nkv) * hd)
        if parts & 4:
            dqkv[:, :nh * hd].copy_(q.grad.reshape(T, -1))
        if parts & 2:
            dqkv[:, nh * hd:].copy_(torch.cat([kk.grad.reshape(T, -1), v.grad.reshape(T, -1)], 1))

    def _k_swiglu_fwd(self, r, x):
        T, F = x.i[0], x.i[1]
        gu = r.mat(x.t[0], T, 2 * F).float()
        g, u = gu[:, :F], gu[:, F:]
        r.mat(x.t[1], T, F).copy_(g * torch.sigmoid(g) * u)

    def _k_swiglu_bwd(self, r, x):
        T, F = x.i[0], x.i[1]
        gu, da = r.mat(x.t[0], T, 2 * F).float(), r.mat(x.t[1], T, F).float()
        g, u = gu[:, :F], gu[:, F:]
        sg = torch.sigmoid(g)
        r.mat(x.t[2], T, 2 * F).copy_(torch.cat([da * u * sg * (1 + g * (1 - sg)), da * g * sg], 1))

    def _k_cross_entropy(self, r, x):
        rows, V = x.i[0], x.i[1]
        lg = r.mat(x.t[0], rows, V)
        tgt = r.flat(x.t[1], rows).long()
        z = lg.float()
        lse = torch.logsumexp(z, -1)
        live = tgt >= 0
        safe = tgt.clamp(min=0)
        loss = (lse - z.gather(1, safe[:, None])[:, 0])[live].sum()
        d = torch.softmax(z, -1)
        d[torch.arange(rows), safe] -= 1.0
        d[~live] = 0.0
        lg.copy_(d * float(x.f[0]))
        acc = r.flat(x.t[2], 1)
        acc.copy_(acc + loss * float(x.f[1]))

    def _k_adamw(self, r, x):
        n = (int(x.i[1]) & 0xFFFFFFFF) << 32 | (int(x.i[0]) & 0xFFFFFFFF)
        self._adamw(r.flat(x.t[0], n), r.flat(x.t[1], n), r.flat(x.t[2], n), r.flat(x.t[3], n).float() * float(x.f[0]),
                    [r.flat(x.t[4], n)])

    def _adamw(self, master, m, v, g, params):
        lr, b1, b2, eps, wd, bc1, bc2 = self.hyper
        m.copy_(b1 * m + (1 - b1) * g)
        v.copy_(b2 * v + (1 - b2) * g * g)
        master.copy_(master - lr * ((m / bc1) / ((v / bc2).sqrt() + eps) + wd * master))
        for p in params:
            p.copy_(master)

    def _k_zero(self, r, x):
        t = r.pf.tensors[x.t[0]]
        r.arena[t.offset:t.offset + t.nbytes].zero_()

    def _k_add(self, r, x):
        n = x.i[0]
        r.flat(x.t[2], n).copy_(r.flat(x.t[0], n).float() + r.flat(x.t[1], n).float())

    def _k_moe_route(self, r, x):
        T, E, k = x.i[0], x.i[1], x.i[2]
        logits = r.mat(x.t[0], T, E).float()
        if x.flags & 1:     # backward: dlogits from the gradient of the renormalised top-k weights
            idx, pos = r.mat(x.t[1], T, k).long(), r.mat(x.t[3], T, k)
            z = logits.clone().requires_grad_(True)
            p = torch.softmax(z, -1).gather(1, idx)
            w = p / p.sum(-1, keepdim=True)
            dw = torch.where(pos >= 0, r.mat(x.t[2], T, k).float(), torch.zeros(()))     # dropped choices carry no gradient
            w.backward(dw)
            r.mat(x.t[4], T, E).copy_(z.grad)
            return
        cap = x.i[3]
        p = torch.softmax(logits, -1)
        # top-k, ties to the lower index (a stable descending sort does that)
        order = torch.sort(p, dim=-1, descending=True, stable=True)
        idx, top = order.indices[:, :k], order.values[:, :k]
        r.mat(x.t[1], T, k).copy_(idx)
        r.mat(x.t[2], T, k).copy_(top / top.sum(-1, keepdim=True))
        # slot of every (token, choice) in its expert's slab, in token order; -1 past the capacity
        flat = idx.reshape(-1)
        counts = torch.bincount(flat, minlength=E)
        order = torch.argsort(flat, stable=True)                     # entries grouped by expert, token order kept
        first = torch.cumsum(counts, 0) - counts                      # where each expert's group starts
        slot = torch.empty_like(flat)
        slot[order] = torch.arange(flat.numel()) - first[flat[order]]
        pos = torch.where(slot < cap, slot, torch.full_like(slot, -1))
        r.mat(x.t[3], T, k).copy_(pos.view(T, k))
        r.flat(x.t[4], E).copy_(counts)

    # ------------------------------------------------------------------ records of a whole group
    def _g_moe_dispatch(self, ranks, xs):
        """Every member permutes its rows by expert straight into the owners' slabs: slab (local expert, source member),
        row = the slot the router gave; the owners also learn how many rows each source sent."""
        x0 = xs[0]
        k, E, cap = x0.i[0], x0.i[1], x0.i[2]
        n = len(ranks)
        E_l = E // n
        for src, (r, x) in enumerate(zip(ranks, xs)):
            T, H, _ = r.pf.shape(x.t[0])
            rows = r.mat(x.t[0], T, H).float()
            idx, pos = r.mat(x.t[1], T, k).long(), r.mat(x.t[2], T, k).long()
            scale = r.mat(x.t[3], T, k).float() if x.t[3] >= 0 else None
            counts = r.flat(x.t[4], E).long()
            for e in range(E):
                owner, el = e // E_l, e % E_l
                o, ox = ranks[owner], xs[owner]
                sub = el * n + src
                cnt = min(int(counts[e]), cap)
                o.flat(ox.t[6], E_l * n)[sub] = cnt
                slab = o.mat(ox.t[5], E_l * n * cap, H)
                slab[sub * cap + cnt:(sub + 1) * cap].zero_()          # the device zeroes up to the next 128; rows past a count are never read
                sel = (idx == e) & (pos >= 0)
                t_i, s_i = torch.nonzero(sel, as_tuple=True)
                if t_i.numel():
                    v = rows[t_i] * (scale[t_i, s_i][:, None] if scale is not None else 1.0)
                    slab[sub * cap + pos[t_i, s_i]] = v.to(slab.dtype)

    def _g_moe_combine(self, ranks, xs):
        """Every member pulls the rows of its tokens back out of the owners' slabs: weighted sum onto a base, plain sum,
        or (dw mode) the dot product of each row with the token's incoming gradient."""
        x0 = xs[0]
        k, E, cap = x0.i[0], x0.i[1], x0.i[2]
        n = len(ranks)
        E_l = E // n
        for me, (r, x) in enumerate(zip(ranks, xs)):
            T = r.pf.shape(x.t[2])[0]
            H = r.pf.shape(x.t[5])[1]
            idx, pos = r.mat(x.t[2], T, k).long(), r.mat(x.t[3], T, k).long()
            w = r.mat(x.t[4], T, k).float() if x.t[4] >= 0 else torch.ones(T, k)
            got = torch.zeros(T, k, H)
            for owner in range(n):
                slab = ranks[owner].mat(xs[owner].t[5], E_l * n * cap, H).float()
                sel = (idx // E_l == owner) & (pos >= 0)
                t_i, s_i = torch.nonzero(sel, as_tuple=True)
                if t_i.numel():
                    got[t_i, s_i] = slab[((idx[t_i, s_i] % E_l) * n + me) * cap + pos[t_i, s_i]]
            if x.t[7] >= 0:
                r.mat(x.t[7], T, k).copy_((got * r.mat(x.t[6], T, H).float()[:, None, :]).sum(-1))
                continue
            out = (got * w[:, :, None]).sum(1)
            if x.t[0] >= 0:
                out = out + r.mat(x.t[0], T, H).float()
            r.mat(x.t[1], T, H).copy_(out)

    @staticmethod
    def _count(x):
        return (int(x.i[1]) & 0xFFFFFFFF) << 32 | (int(x.i[0]) & 0xFFFFFFFF)

    def _g_all_reduce(self, ranks, xs):
        n = self._count(xs[0])
        total = sum(r.flat(x.t[0], n).float() for r, x in zip(ranks, xs))
        for r, x in zip(ranks, xs):
            r.flat(x.t[1], n).copy_(total)

    def _g_reduce_scatter(self, ranks, xs):
        n = self._count(xs[0])                          # elements every member receives
        srcs = [r.flat(x.t[0], n * len(ranks)).float() for r, x in zip(ranks, xs)]
        for i, (r, x) in enumerate(zip(ranks, xs)):
            r.flat(x.t[1], n).copy_(sum(s[i * n:(i + 1) * n] for s in srcs))

    def _g_all_gather(self, ranks, xs):
        n = self._count(xs[0])                          # elements every member contributes
        parts = [r.flat(x.t[0], n).clone() for r, x in zip(ranks, xs)]
        for r, x in zip(ranks, xs):
            dst = r.flat(x.t[1], n * len(ranks))
            for i, p in enumerate(parts):
                dst[i * n:(i + 1) * n].copy_(p)

    def _g_cross_entropy_tp(self, ranks, xs):
        rows, Vl = xs[0].i[0], xs[0].i[1]
        z = [r.mat(x.t[0], rows, Vl).float() for r, x in zip(ranks, xs)]
        full = torch.cat(z, 1)
        lse = torch.logsumexp(full, -1)
        for (r, x), zl in zip(zip(ranks, xs), z):
            lo = x.i[2]
            tgt = r.flat(x.t[1], rows).long()
            live = tgt >= 0
            mine = live & (tgt >= lo) & (tgt < lo + Vl)
            d = torch.exp(zl - lse[:, None])
            idx = torch.nonzero(mine)[:, 0]
            d[idx, tgt[idx] - lo] -= 1.0
            d[~live] = 0.0
            loss = -zl[idx, tgt[idx] - lo].sum()
            if x.i[4]:
                loss = loss + lse[live].sum()
            r.mat(x.t[0], rows, Vl).copy_(d * float(x.f[0]))
            acc = r.flat(x.t[2], 1)
            acc.copy_(acc + loss * float(x.f[1]))

    def _g_ag_gemm(self, ranks, xs):
        x0 = xs[0]
        T, N, Kd = x0.i[0], x0.i[1], x0.i[2]
        Tl = T // len(ranks)
        blocks = [r.mat(x.t[0], Tl, Kd).clone() for r, x in zip(ranks, xs)]
        for r, x in zip(ranks, xs):
            full = r.mat(x.t[3], T, Kd)
            for i, b in enumerate(blocks):
                full[i * Tl:(i + 1) * Tl].copy_(b)
            tb, epi = (x.flags >> 1) & 1, (x.flags >> 4) & 0xF
            acc = self._gemm_core(r, x.t[3], x.t[1], T, N, Kd, 0, tb)
            self._epilogue(r, acc, x, x.t[2], x.t[5], epi)

    def _g_gemm_rs(self, ranks, xs):
        x0 = xs[0]
        T, N, Kd = x0.i[0], x0.i[1], x0.i[2]
        Tl = T // len(ranks)
        # partial products travel as bf16 (the staging buffers of the kernel), the owner sums them in fp32
        partial = [self._gemm_core(r, x.t[0], x.t[1], T, N, Kd, 0, (x.flags >> 1) & 1).to(torch.bfloat16).float()
                   for r, x in zip(ranks, xs)]
        for i, (r, x) in enumerate(zip(ranks, xs)):
            total = sum(p[i * Tl:(i + 1) * Tl] for p in partial)
            if x.t[3] >= 0:
                total = total + r.mat(x.t[3], Tl, N).float()
            r.mat(x.t[2], Tl, N).copy_(total)

    def _g_fsdp_gather(self, ranks, xs):
        """ZeRO-3: the flat range [lo, hi) of the parameter space, whose member r keeps [r * n_shard, (r + 1) * n_shard),
        lands in every member's staging buffer (fused into the GEMM that follows it on the device, or a kernel of its own)."""
        x0 = xs[0]
        lo, hi = (int(x0.i[0]) & 0xFFFFFFFF) << 9, (int(x0.i[1]) & 0xFFFFFFFF) << 9
        n_shard = ranks[0].rl.n_shard
        whole = torch.cat([r.flat(x.t[0])[:n_shard] for r, x in zip(ranks, xs)])
        for r, x in zip(ranks, xs):
            r.flat(x.t[1], hi - lo).copy_(whole[lo:hi])

    def _g_rs_adamw(self, ranks, xs):
        x0 = xs[0]
        gscale = float(x0.f[0])
        own_params, staged = bool(x0.flags & 1), bool(x0.flags & 4)      # ZeRO-3: parameters / gradients sharded too
        acc_only, acc_first = bool(x0.flags & 8), bool(x0.flags & 16)
        if x0.flags & 2:        # a bucket [lo, hi) of the flat space; the kernel indexes from the flat buffers
            lo, hi = (int(x0.i[0]) & 0xFFFFFFFF) << 9, (int(x0.i[1]) & 0xFFFFFFFF) << 9
            n_flat, n_shard = ranks[0].rl.n_rep, ranks[0].rl.n_shard
            names = ("@flat_master", "@flat_m", "@flat_v", "@flat_grad", "@flat_param")
            buf = [[r.named_flat(n) for n in names] for r in ranks]
            if staged:          # one microbatch's gradients of the bucket, element i of the flat space at i - lo
                for b, (r, x) in zip(buf, zip(ranks, xs)):
                    b[3] = r.flat(x.t[3])
        else:
            n_flat = (int(x0.i[1]) & 0xFFFFFFFF) << 32 | (int(x0.i[0]) & 0xFFFFFFFF)
            n_shard = int(x0.i[2]) & 0xFFFFFFFF
            lo, hi = 0, n_flat
            buf = [[r.flat(x.t[j]) for j in range(5)] for r, x in zip(ranks, xs)]
        for i, (r, x) in enumerate(zip(ranks, xs)):
            s_lo = i * n_shard
            first, last = max(s_lo, lo), min(min(s_lo + n_shard, n_flat), hi)
            if first >= last:
                continue
            g0 = lo if staged else 0
            g = sum(b[3][first - g0:last - g0].float() for b in buf)
            if staged and x.t[5] >= 0:      # running sum over the microbatches, kept by the owner
                gacc = r.flat(x.t[5])[:last - first]
                if not acc_first:
                    g = g + gacc
                if acc_only:
                    gacc.copy_(g)
                    continue
            master, m, v = (buf[i][j][first - s_lo:last - s_lo] for j in range(3))
            params = [buf[i][4][first - s_lo:last - s_lo]] if own_params else [b[4][first:last] for b in buf]
            self._adamw(master, m, v, g * gscale, params)

    _local = {K["gemm"]: _k_gemm, K["embed_fwd"]: _k_embed_fwd, K["embed_bwd"]: _k_embed_bwd, K["rmsnorm_fwd"]: _k_rmsnorm_fwd,
              K["rmsnorm_bwd"]: _k_rmsnorm_bwd, K["rope"]: _k_rope, K["attn_fwd"]: _k_attn_fwd, K["attn_bwd"]: _k_attn_bwd,
              K["swiglu_fwd"]: _k_swiglu_fwd, K["swiglu_bwd"]: _k_swiglu_bwd, K["cross_entropy"]: _k_cross_entropy,
              K["adamw"]: _k_adamw, K["zero"]: _k_zero, K["add"]: _k_add, K["quant_fp8"]: _k_quant_fp8, K["gemm_fp8"]: _k_gemm_fp8,
              K["moe_route"]: _k_moe_route}
    _group_ops = {K["nccl_all_reduce"]: _g_all_reduce, K["nccl_reduce_scatter"]: _g_reduce_scatter,
                  K["nccl_all_gather"]: _g_all_gather, K["cross_entropy_tp"]: _g_cross_entropy_tp, K["ag_gemm"]: _g_ag_gemm,
                  K["gemm_rs"]: _g_gemm_rs, K["rs_adamw"]: _g_rs_adamw, K["fsdp_ag_gemm"]: _g_fsdp_gather,
                  K["moe_dispatch_gemm"]: _g_moe_dispatch, K["moe_gemm_combine"]: _g_moe_combine}


def random_state(interp: PlanInterpreter, seed=0, std=0.02):
    """A global parameter state (master drawn N(0, std), gains 1, moments 0) shaped after the job's own tables."""
    g = np.random.default_rng(seed)
    state = {}
    for rl in interp.layouts():
        for name, _, rows, cols in rl.params:
            if name in state:
                continue
            gshape, _ = rl.slice_of(name, rows, cols)
            gain = name.split(".")[-1] in ("g1", "g2", "gf")
            master = np.ones(gshape, dtype=np.float32) if gain else (g.standard_normal(gshape) * std).astype(np.float32)
            state[name] = {"master": master, "m": np.zeros(gshape, dtype=np.float32), "v": np.zeros(gshape, dtype=np.float32)}
    return state


def check_against_reference(config_text: str, steps: int = 3, seed: int = 1, order: str = "program"):
    """Trains the interpreted job and the one-device fp32 model (``reference_torch.forward_loss`` + AdamW on fp32 master
    weights read as bf16, like the kernels read them) on the same random batches from the same random parameters.
    Returns ``(losses, drift)``: per step ``(interpreted, reference)``, and the largest mean distance between the two
    runs' master parameters relative to how far the parameter moved (a few percent for a correct layout: bf16 storage
    turns some near-zero gradients around; a wrong shard or a lost contribution moves whole tensors)."""
    from . import reference_torch as ref
    it = PlanInterpreter(config_text, order=order, seed=seed)
    st = random_state(it, seed=seed)
    it.load_state(st)
    m, tr = it.model, it.train
    master = {k: torch.tensor(v["master"]).clone() for k, v in st.items()}
    start = {k: v.clone() for k, v in master.items()}
    mom = {k: torch.zeros_like(v) for k, v in master.items()}
    var = {k: torch.zeros_like(v) for k, v in master.items()}
    G, S = it.rows_per_replica * int(it.hdr.dp), int(m.seq_len)
    gen = torch.Generator().manual_seed(5)
    losses = []
    for step in range(1, steps + 1):
        tok = torch.randint(0, m.vocab_size, (G, S), generator=gen)
        tgt = torch.randint(0, m.vocab_size, (G, S), generator=gen)
        got = it.step(tok, tgt)
        p = {k: v.to(torch.bfloat16).float().requires_grad_(True) for k, v in master.items()}
        loss = ref.forward_loss(p, tok, tgt, layers=m.num_layers, heads=m.num_heads, kv_heads=m.num_kv_heads,
                                head_dim=m.head_dim, seq=S, eps=tr.norm_eps, theta=tr.rope_theta,
                                top_k=int(m.moe_top_k) if m.is_moe else 0)
        loss.backward()
        b1, b2 = tr.beta1, tr.beta2
        for k in master:
            g = p[k].grad
            mom[k] = b1 * mom[k] + (1 - b1) * g
            var[k] = b2 * var[k] + (1 - b2) * g * g
            master[k] = master[k] - tr.lr * ((mom[k] / (1 - b1 ** step)) / ((var[k] / (1 - b2 ** step)).sqrt() + tr.adam_eps)
                                             + tr.weight_decay * master[k])
        losses.append((got, float(loss.detach())))
    end = it.state()
    drift = max(float((torch.tensor(end[k]["master"]) - master[k]).abs().mean() / ((master[k] - start[k]).abs().mean() + 1e-12))
                for k in master)
    return losses, drift


def main(argv=None):
    """``python -m cai_b200.models.plan_interpreter CONFIG [--steps N] [--order random]``: before a layout goes to the
    GPUs, run its executable plans on the host, every rank in this process, next to the one-device fp32 model. Meant
    for small stand-ins of the real model (same layout keys, small sizes): the arenas of all ranks live in host memory."""
    import argparse
    ap = argparse.ArgumentParser(description="interpret a configuration's executable plans on the host and compare with the fp32 model")
    ap.add_argument("config")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--order", choices=("program", "random"), default="program",
                    help="random: any interleaving of a rank's streams that the plan's events allow")
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--tolerance", type=float, default=5e-3, help="largest accepted |interpreted - reference| loss")
    a = ap.parse_args(argv)
    planlib.set_log_level("warn")
    losses, drift = check_against_reference(Path(a.config).read_text(), a.steps, a.seed, a.order)
    worst = 0.0
    for i, (got, want) in enumerate(losses, 1):
        print(f"step {i}: interpreted {got:.5f}   fp32 model {want:.5f}   difference {got - want:+.5f}")
        worst = max(worst, abs(got - want))
    ok = worst <= a.tolerance and drift < 0.5
    print(f"parameters apart by {drift * 100:.1f}% of the distance they moved; " + ("PASS" if ok else "FAIL"))
    return 0 if ok else 1


if __name__ == "__main__":
    raise SystemExit(main())
