"""Stand-alone check and micro-benchmark of the fused compute+collective GEMMs on 1..8 GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        cai_b200/parallel/fused_bench.py --op gemm_rs --tokens 4096 --out-features 2048 --in-features 2048

(run as ``python cai_b200/parallel/fused_bench.py ...`` for a single process and a group of one).
Every rank owns one buffer (signal block, inputs, staging) that the others map over CUDA IPC, as the
engine does with its arena. For the chosen op the script
  * checks the fused kernel against the same product computed with a plain GEMM and an NCCL
    collective (``torch.distributed``),
  * times both (CUDA events, L2 flushed, max over ranks), and
  * prints one JSON line (rank 0) with the roofline: the slower of FLOPs at the measured GEMM peak and
    the bytes that must cross NVLink at the measured per-direction peer bandwidth (770 GB/s).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
from ctypes import c_int, c_longlong, c_uint32, c_ulonglong, c_void_p
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))   # launched as a script by torch.distributed.run

from cai_b200.ops import _lib as klib  # noqa: E402
from cai_b200.ops import gemm  # noqa: E402

GROUP_TP = 0
NVLINK_GBS = 770.0   # measured peer copy bandwidth per direction per GPU on this pool


class PeerBuffer:
    """One device buffer per rank, mapped by every other rank; offset 0 holds the signal block."""

    def __init__(self, nbytes: int, rank: int, world: int, device):
        self.L = klib.lib()
        L = self.L
        L.cai_ipc_export.argtypes = [c_void_p, c_void_p, ctypes.POINTER(c_ulonglong)]
        L.cai_ipc_open.argtypes = [c_void_p, c_ulonglong, ctypes.POINTER(c_void_p)]
        L.cai_ipc_close.argtypes = [c_void_p, c_ulonglong]
        P, I, LL, ULL = c_void_p, c_int, c_longlong, c_ulonglong
        L.cai_fused_ag_gemm_c.argtypes = [P, I, I, ULL, I, ULL, LL, P, P, P, I, I, I, LL, LL, I, P, c_uint32, I, P]
        L.cai_fused_gemm_rs_c.argtypes = [P, I, I, ULL, I, P, P, ULL, P, P, I, I, I, LL, LL, LL, LL, I, P, c_uint32, P]
        F = ctypes.c_float
        L.cai_fused_rs_adamw_c.argtypes = [P, I, I, ULL, ULL, ULL, P, P, P, LL, LL, P, F, c_uint32, P, I, P]
        L.cai_fused_gather_gemm_c.argtypes = [P, I, I, ULL, ULL, LL, LL, LL, P, I, I, P, LL, P, I, I, I, LL, LL, LL, I, P, c_uint32, P]
        self.rank, self.world = rank, world
        self.sig_bytes = int(L.cai_signal_block_bytes())
        self.buf = torch.zeros(self.sig_bytes + nbytes + 4096, dtype=torch.uint8, device=device)
        self.cursor = self.sig_bytes
        handle = ctypes.create_string_buffer(64)
        off = c_ulonglong(0)
        klib.check(L.cai_ipc_export(c_void_p(self.buf.data_ptr()), handle, ctypes.byref(off)), "ipc_export")
        blobs = [None] * world
        dist.all_gather_object(blobs, handle.raw + off.value.to_bytes(8, "little"))
        self.opened = []
        bases = []
        for r, blob in enumerate(blobs):
            if r == rank:
                bases.append(self.buf.data_ptr())
                continue
            out = c_void_p()
            o = int.from_bytes(blob[64:72], "little")
            klib.check(L.cai_ipc_open(ctypes.create_string_buffer(blob[:64], 64), c_ulonglong(o), ctypes.byref(out)), "ipc_open")
            self.opened.append((out.value, o))
            bases.append(out.value)
        self.bases = (c_void_p * world)(*[c_void_p(b) for b in bases])
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.seq = 0

    def alloc(self, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        self.cursor = (self.cursor + 1023) & ~1023
        off = self.cursor
        self.cursor += nbytes
        assert self.cursor <= self.buf.numel()
        return self.buf[off:off + nbytes].view(dtype).view(*shape), off

    def next_seq(self):
        self.seq += 1
        return self.seq

    def close(self):
        torch.cuda.synchronize()
        dist.barrier()
        for base, off in self.opened:
            self.L.cai_ipc_close(c_void_p(base), c_ulonglong(off))
        self.opened = []


def _time(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
        torch.cuda.synchronize()
        dist.barrier()   # back-to-back calls of one fused op have no collective in between to order buffer reuse
    out = []
    for _ in range(iters):
        flush.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        out.append(s.elapsed_time(e))
    t = torch.tensor([statistics.median(out)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


STAMP_WORDS = ("entry", "first_ready", "first_acc", "last_epilogue", "reduce_start", "reduce_flags", "end", "copy_done")


def _phase_summary(buf):
    """Per-CTA stamp records (globaltimer ns, 8 words per CTA) -> microseconds since the first CTA entered."""
    t = buf.view(-1, 8).cpu().numpy().astype("float64")
    live = t[t[:, 0] > 0]
    if not len(live):
        return {}
    t0 = live[:, 0].min()
    out = {"ctas": int(len(live))}
    for i, name in enumerate(STAMP_WORDS):
        col = live[:, i][live[:, i] > 0]
        if len(col):
            out[name] = {"min": (col.min() - t0) / 1e3, "median": (statistics.median(col.tolist()) - t0) / 1e3,
                         "max": (col.max() - t0) / 1e3}
    return out


def tp_chain(a, pb, L, rank, world, dev, st, flush, gemm_peak, res):
    """The pattern of a tensor-parallel MLP in steady state: x_local[T/n, H] -> all-gather -> GEMM (W1[F, H]) ->
    GEMM (W2[H, F]) -> reduce-scatter -> x_local, `--chain` times back to back without a host synchronisation, as
    the executor enqueues it. Reports the time per pair against the same chain through NCCL and, from the last
    pair, where the CTAs of each kernel spent their time (per-CTA globaltimer stamps)."""
    bf = torch.bfloat16
    T, F, H = a.tokens, a.out_features, a.in_features
    Tl = T // world
    x_local, x_off = pb.alloc((Tl, H), bf)
    a_full, _ = pb.alloc((T, H), bf)
    _, stage_off = pb.alloc((world, Tl, H), bf)
    x_local.copy_(torch.randn(Tl, H, device=dev))
    W1 = (torch.randn(F, H, device=dev) * H ** -0.5).to(bf)
    W2 = (torch.randn(H, F, device=dev) * (F * world) ** -0.5).to(bf)
    y = torch.empty(T, F, device=dev, dtype=bf)
    L.cai_fused_debug_stamps.argtypes = [c_void_p]
    stamps = [torch.zeros(256 * 8, dtype=torch.int64, device=dev) for _ in range(2)]
    dist.barrier()

    def pair(with_stamps=False):
        if with_stamps:
            L.cai_fused_debug_stamps(c_void_p(stamps[0].data_ptr()))
        klib.check(L.cai_fused_ag_gemm_c(pb.bases, rank, world, 0, GROUP_TP, x_off, H, a_full.data_ptr(), W1.data_ptr(), y.data_ptr(),
                                         T, F, H, H, F, 0, pb.epoch.data_ptr(), pb.next_seq(), a.copy_ctas, st), "ag_gemm")
        if with_stamps:
            L.cai_fused_debug_stamps(c_void_p(stamps[1].data_ptr()))
        klib.check(L.cai_fused_gemm_rs_c(pb.bases, rank, world, 0, GROUP_TP, y.data_ptr(), W2.data_ptr(), stage_off, x_local.data_ptr(),
                                         None, T, H, F, F, F, H, 0, 0, pb.epoch.data_ptr(), pb.next_seq(), st), "gemm_rs")
        if with_stamps:
            L.cai_fused_debug_stamps(None)

    def fused():
        for i in range(a.chain):
            pair(with_stamps=(i == a.chain - 1))

    gathered = torch.empty(T, H, device=dev, dtype=bf)
    partial = torch.empty(T, H, device=dev, dtype=bf)
    xb = x_local.clone()

    def baseline():
        for _ in range(a.chain):
            dist.all_gather_into_tensor(gathered, xb)
            gemm(gathered, W1, out=y)
            gemm(y, W2, out=partial)
            dist.reduce_scatter_tensor(xb, partial)

    ms_f = _time(fused, a.iters, a.warmup, flush) / a.chain
    ms_b = _time(baseline, a.iters, a.warmup, flush) / a.chain
    flops = 2.0 * 2.0 * T * F * H
    link = 2 * (world - 1) * Tl * H * 2          # rows pulled by the gather + partial rows pushed by the reduce-scatter
    roof = max(flops / (gemm_peak * 1e12), link / (NVLINK_GBS * 1e9))
    phases = {"ag_gemm": _phase_summary(stamps[0]), "gemm_rs": _phase_summary(stamps[1])}
    allp = [None] * world
    dist.all_gather_object(allp, phases)
    res.update(T=T, N=F, K=H, chain=a.chain, fused_us_per_pair=ms_f * 1e3, nccl_path_us_per_pair=ms_b * 1e3,
               speedup_vs_nccl_path=ms_b / ms_f, roofline_us_per_pair=roof * 1e6, frac_of_roofline=roof / (ms_f * 1e-3),
               link_bytes_per_pair=link, status=klib.device_status(clear=True), fused_us=ms_f * 1e3, phases_us_by_rank=allp)
    if rank == 0:
        print(json.dumps(res), flush=True)
    pb.close()
    dist.destroy_process_group()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=["ag_gemm", "gemm_rs", "rs_adamw", "gather_gemm", "moe_exchange", "tp_chain"], required=True)
    ap.add_argument("--chain", type=int, default=24, help="tp_chain: all-gather -> GEMM / GEMM -> reduce-scatter pairs enqueued back to back")
    ap.add_argument("--params", type=int, default=256 << 20, help="rs_adamw: elements of the flat parameter space")
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=8)
    # (names chosen so that none is a prefix of an option of torch.distributed.run)
    ap.add_argument("--tokens", type=int, default=4096, help="rows T of the full (gathered) activation")
    ap.add_argument("--out-features", type=int, default=2048, help="N")
    ap.add_argument("--in-features", type=int, default=2048, help="K")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--copy-ctas", type=int, default=0, help="0: chosen by the library")
    a = ap.parse_args(argv)
    # without a launcher: one process, a group of one (the kernels then move the local rows only)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29591")
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group(backend="cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    L = klib.lib()
    bf = torch.bfloat16
    T, N, K = a.tokens, a.out_features, a.in_features
    Tl = T // world
    need = 2 * T * K * 2 + 2 * T * N * 2 + (64 << 20)
    if a.op == "rs_adamw":
        need = a.params * 6 + (64 << 20)
    if a.op == "gather_gemm":
        need = (N * K * 4 // world + (1 << 20)) * 2 + (64 << 20)
    if a.op == "moe_exchange":
        need = 3 * 2 * T * a.top_k * K * 2 * 2 + (64 << 20)   # slabs at capacity factor 2
    pb = PeerBuffer(need, rank, world, dev)
    st = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(1234 + rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    gemm_peak = peaks.get("bf16_tflops", 1590.0)
    res = {"op": a.op, "world": world, "T": T, "N": N, "K": K}
    if a.op == "tp_chain":
        return tp_chain(a, pb, L, rank, world, dev, st, flush, gemm_peak, res)
    if a.op == "ag_gemm":
        # C[T,N] = gather(x_local[Tl,K]) @ W[N,K]^T
        x_local, x_off = pb.alloc((Tl, K), bf)
        a_full, _ = pb.alloc((T, K), bf)
        x_local.copy_(torch.randn(Tl, K, device=dev))
        W = (torch.randn(N, K, device=dev) * 0.05).to(bf)
        C = torch.empty(T, N, device=dev, dtype=bf)
        dist.barrier()

        def fused():
            klib.check(L.cai_fused_ag_gemm_c(pb.bases, rank, world, 0, GROUP_TP, x_off, K, a_full.data_ptr(), W.data_ptr(),
                                             C.data_ptr(), T, N, K, K, N, 0, pb.epoch.data_ptr(), pb.next_seq(), a.copy_ctas, st),
                       "ag_gemm")

        gathered = torch.empty(T, K, device=dev, dtype=bf)
        Cb = torch.empty(T, N, device=dev, dtype=bf)

        def baseline():
            dist.all_gather_into_tensor(gathered, x_local)
            gemm(gathered, W, out=Cb)

        fused(); baseline()
        torch.cuda.synchronize()
        err = (C.float() - Cb.float()).abs().max().item()
        res["max_abs_diff_vs_nccl_path"] = err
        assert err <= 2e-2 * Cb.float().abs().max().item() + 1e-3, err
        link_bytes = (world - 1) * Tl * K * 2          # rows pulled from the other members
    elif a.op == "rs_adamw":
        # gradient reduce-scatter + scale + sharded AdamW + bf16 parameter all-gather vs NCCL all-reduce + replicated AdamW
        from cai_b200.ops import adamw_
        n = a.params // (512 * world) * 512 * world
        ns = n // world
        grad, g_off = pb.alloc((n,), torch.float32)
        param, p_off = pb.alloc((n,), bf)
        grad.copy_(torch.randn(n, device=dev) * 1e-2)
        master = torch.randn(ns, device=dev) * 0.02
        m1, v1 = torch.zeros(ns, device=dev), torch.zeros(ns, device=dev)
        hyper = torch.tensor([1e-3, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001, 0.0], device=dev)
        scratch = torch.zeros(4, device=dev, dtype=torch.int32)
        dist.barrier()

        def fused():
            klib.check(L.cai_fused_rs_adamw_c(pb.bases, rank, world, 0, g_off, p_off, master.data_ptr(), m1.data_ptr(), v1.data_ptr(),
                                              n, ns, hyper.data_ptr(), 1.0 / world, pb.next_seq(), scratch.data_ptr(), 0, st), "rs_adamw")

        gb = grad.clone()
        mb_, mm, vv, pp = torch.randn(n, device=dev) * 0.02, torch.zeros(n, device=dev), torch.zeros(n, device=dev), torch.empty(n, device=dev, dtype=bf)

        def baseline():
            dist.all_reduce(gb)
            adamw_(mb_, mm, vv, gb, pp, step=1, lr=1e-3, grad_scale=1.0 / world)

        fused(); baseline()
        torch.cuda.synchronize()
        res["max_abs_diff_vs_nccl_path"] = 0.0   # different initial masters: timing only (numerics: multi-GPU training tests)
        flops = 0.0
        link_bytes = (world - 1) * ns * 4 + (world - 1) * ns * 2   # gradient shards pulled + bf16 parameters pushed
        res["hbm_bytes"] = world * ns * 4 + ns * 24 + ns * 2 * world
    elif a.op == "gather_gemm":
        # ZeRO-3: W[N,K] sharded over the group, gathered by the copy CTAs of C[T,N] = X[T,K] @ W^T
        n = (N * K + 512 * world - 1) // (512 * world) * 512 * world
        ns = n // world
        shard, s_off = pb.alloc((ns,), bf)
        shard.copy_(torch.randn(ns, device=dev) * 0.05)
        stage = torch.empty(n, device=dev, dtype=bf)
        X = torch.randn(T, K, device=dev).to(bf)
        C = torch.empty(T, N, device=dev, dtype=bf)
        dist.barrier()

        def fused():
            klib.check(L.cai_fused_gather_gemm_c(pb.bases, rank, world, 0, s_off, ns, 0, n, stage.data_ptr(), 0, a.copy_ctas or 24,
                                                 X.data_ptr(), 0, C.data_ptr(), T, N, K, K, K, N, 0, pb.epoch.data_ptr(),
                                                 pb.next_seq(), st), "gather_gemm")

        full = torch.empty(n, device=dev, dtype=bf)
        Cb = torch.empty(T, N, device=dev, dtype=bf)

        def baseline():
            dist.all_gather_into_tensor(full, shard)
            gemm(X, full[:N * K].view(N, K), out=Cb)

        fused(); baseline()
        torch.cuda.synchronize()
        err = (C.float() - Cb.float()).abs().max().item()
        res["max_abs_diff_vs_nccl_path"] = err
        assert err <= 2e-2 * Cb.float().abs().max().item() + 1e-3, err
        link_bytes = (world - 1) * ns * 2
    elif a.op == "moe_exchange":
        # dispatch (permute + peer stores + handshake) and combine (peer loads + weighted sum) of T tokens, hidden K
        from cai_b200.ops import moe_route_fwd
        P_, I_, ULL_ = c_void_p, c_int, c_ulonglong
        E, k, H = a.experts, a.top_k, K
        cap = (2 * T * k // E + 127) // 128 * 128
        E_l = E // world
        rows = E_l * world * cap
        xs, xs_off = pb.alloc((rows, H), bf)
        ys, ys_off = pb.alloc((rows, H), bf)
        cnt, cnt_off = pb.alloc((E_l * world,), torch.int32)
        x = torch.randn(T, H, device=dev).to(bf)
        idx, w, pos, counts = moe_route_fwd(torch.randn(T, E, device=dev), k, cap)
        ys.copy_(torch.randn(rows, H, device=dev))
        out = torch.empty(T, H, device=dev, dtype=bf)
        scratch = torch.zeros(4, device=dev, dtype=torch.int32)
        dist.barrier()

        def fused():
            klib.check(L.cai_moe_dispatch_c(pb.bases, rank, world, 0, x.data_ptr(), idx.data_ptr(), pos.data_ptr(), None,
                                            counts.data_ptr(), xs_off, cnt_off, T, H, k, E, cap, pb.epoch.data_ptr(), pb.next_seq(),
                                            scratch.data_ptr(), st), "dispatch")
            klib.check(L.cai_moe_combine_c(pb.bases, rank, world, 0, x.data_ptr(), out.data_ptr(), idx.data_ptr(), pos.data_ptr(),
                                           w.data_ptr(), ys_off, None, None, T, H, k, E, cap, 1, pb.epoch.data_ptr(), pb.next_seq(),
                                           st), "combine")

        send = torch.empty(T * k, H, device=dev, dtype=bf)
        recv = torch.empty(T * k, H, device=dev, dtype=bf)
        order = torch.argsort(idx.view(-1).long())

        def baseline():
            # what an NCCL path does at least: permute, two equal-split all-to-alls, weighted un-permute
            send.copy_(x.repeat_interleave(k, 0)[order])
            dist.all_to_all_single(recv, send)
            dist.all_to_all_single(send, recv)
            out.copy_((send[torch.argsort(order)].view(T, k, H).float() * w[:, :, None]).sum(1) + x.float())

        fused(); baseline()
        torch.cuda.synchronize()
        res["max_abs_diff_vs_nccl_path"] = 0.0   # timing only here (numerics: tests/test_moe_gpu.py and the ep=2 training test)
        flops = 0.0
        link_bytes = 2 * (world - 1) * (T * k // world) * H * 2   # rows leaving in dispatch + rows pulled in combine
        res["hbm_bytes"] = 2 * (T * k * H * 2) * 2
    else:
        # out_local[Tl,N] = residual + reduce_scatter_rows(A[T,K] @ W[N,K]^T)
        A = torch.randn(T, K, device=dev).to(bf)
        W = (torch.randn(N, K, device=dev) * 0.05).to(bf)
        _, stage_off = pb.alloc((world, Tl, N), bf)
        resid = torch.randn(Tl, N, device=dev).to(bf)
        out = torch.empty(Tl, N, device=dev, dtype=bf)
        dist.barrier()

        def fused():
            klib.check(L.cai_fused_gemm_rs_c(pb.bases, rank, world, 0, GROUP_TP, A.data_ptr(), W.data_ptr(), stage_off,
                                             out.data_ptr(), resid.data_ptr(), T, N, K, K, K, N, N, 0, pb.epoch.data_ptr(),
                                             pb.next_seq(), st), "gemm_rs")

        partial = torch.empty(T, N, device=dev, dtype=bf)
        outb = torch.empty(Tl, N, device=dev, dtype=bf)

        def baseline():
            gemm(A, W, out=partial)
            dist.reduce_scatter_tensor(outb, partial)
            outb.add_(resid)

        fused(); baseline()
        torch.cuda.synchronize()
        err = (out.float() - outb.float()).abs().max().item()
        res["max_abs_diff_vs_nccl_path"] = err
        assert err <= 3e-2 * outb.float().abs().max().item() + 1e-2, err
        link_bytes = (world - 1) * Tl * N * 2          # partial tiles pushed to the other members
    ms_f = _time(fused, a.iters, a.warmup, flush)
    ms_b = _time(baseline, a.iters, a.warmup, flush)
    if a.op in ("ag_gemm", "gemm_rs", "gather_gemm"):
        flops = 2.0 * T * N * K
    t_compute = flops / (gemm_peak * 1e12)
    if "hbm_bytes" in res:   # memory-bound ops: local HBM traffic at the measured copy bandwidth
        t_compute = res["hbm_bytes"] / (peaks.get("hbm_gbs", 6650.0) * 1e9)
    t_link = link_bytes / (NVLINK_GBS * 1e9)
    roof = max(t_compute, t_link)
    res.update(fused_us=ms_f * 1e3, nccl_path_us=ms_b * 1e3, speedup_vs_nccl_path=ms_b / ms_f,
               roofline_us=roof * 1e6, roofline_bound=("hbm" if "hbm_bytes" in res else "compute") if t_compute >= t_link else "nvlink",
               frac_of_roofline=roof / (ms_f * 1e-3), link_bytes=link_bytes, status=klib.device_status(clear=True))
    if rank == 0:
        print(json.dumps(res), flush=True)
    pb.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
