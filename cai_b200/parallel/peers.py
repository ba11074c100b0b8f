"""Peer mapping of arenas for the fused compute+collective kernels.

Every rank exports the CUDA allocation that holds its arena as an IPC handle and publishes it in
the job's key-value store; for each communicator that a fused kernel uses, the members' arenas are
opened (mapped into this process, NVLink peer access enabled) and their base addresses handed to
the native executor. After that any tensor of any member is addressable from inside a kernel as
``base[member] + arena offset``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_ulonglong, c_void_p

from .. import plan as planlib
from ..ops import _lib as klib


def _declare(L):
    if getattr(L, "_cai_peer_declared", False):
        return
    L.cai_ipc_export.argtypes = [c_void_p, c_void_p, ctypes.POINTER(c_ulonglong)]
    L.cai_ipc_open.argtypes = [c_void_p, c_ulonglong, ctypes.POINTER(c_void_p)]
    L.cai_ipc_close.argtypes = [c_void_p, c_ulonglong]
    L.cai_exec_set_peers.argtypes = [c_void_p, c_int, c_int, ctypes.POINTER(c_void_p), c_int]
    L.cai_exec_set_ag_copy_ctas.argtypes = [c_void_p, c_int]
    L.cai_exec_set_ag_copy_ctas.restype = None
    L._cai_peer_declared = True


class PeerArenas:
    """Keeps the mappings of the other ranks' arenas alive for the life of an engine."""

    def __init__(self, engine, store):
        self.engine = engine
        self.L = engine.L
        _declare(self.L)
        self.store = store
        self.opened = {}   # global rank -> (mapped arena base, offset)
        self.key = f"cai/ipc/{engine.hdr.plan_hash:x}"
        base = engine.arena_base
        handle = ctypes.create_string_buffer(64)
        off = c_ulonglong(0)
        klib.check(self.L.cai_ipc_export(c_void_p(base), handle, ctypes.byref(off)), "ipc_export")
        store.set(f"{self.key}/{engine.rank}", handle.raw + off.value.to_bytes(8, "little"))

    def base_of(self, rank: int) -> int:
        if rank == self.engine.rank:
            return self.engine.arena_base
        if rank not in self.opened:
            blob = self.store.get(f"{self.key}/{rank}")
            handle = ctypes.create_string_buffer(blob[:64], 64)
            off = int.from_bytes(blob[64:72], "little")
            out = c_void_p()
            klib.check(self.L.cai_ipc_open(handle, c_ulonglong(off), ctypes.byref(out)), "ipc_open")
            self.opened[rank] = (out.value, off)
        return self.opened[rank][0]

    def attach_group(self, kind: int, members):
        me = members.index(self.engine.rank)
        bases = (c_void_p * len(members))(*[c_void_p(self.base_of(r)) for r in members])
        klib.check(self.L.cai_exec_set_peers(self.engine.ex, kind, len(members), bases, me), "set_peers")

    def close(self):
        for base, off in self.opened.values():
            self.L.cai_ipc_close(c_void_p(base), c_ulonglong(off))
        self.opened.clear()


def expert_group_members(hdr, rank):
    """Members of the expert group of a mixture-of-experts plan under tensor parallelism: the tp ranks of each of
    the ep data-parallel replicas of this rank's block (member index = replica * tp + tp rank). The experts are spread
    over all of them; every member routes the rows of the sequence it owns."""
    tp, ep = int(hdr.tp), max(1, int(hdr.ep))
    replica = tp * int(hdr.num_stages) * int(hdr.cp)
    tp_id, within, dp_id = rank % tp, rank % replica, rank // replica
    first_dp = (dp_id // ep) * ep
    return [within - tp_id + t + (first_dp + i) * replica for i in range(ep) for t in range(tp)]


def attach(engine, groups, store):
    """Exchange arenas for every communicator the plan runs fused kernels on (TP, DP and the expert group)."""
    pa = PeerArenas(engine, store)
    for g in groups:
        if g.kind in (planlib.GROUP_TP, planlib.GROUP_DP) and g.size > 1:
            members = planlib.group_members(engine.config_text, g.kind, engine.rank)
            pa.attach_group(g.kind, members)
    if engine.model.is_moe and engine.hdr.tp > 1:
        pa.attach_group(planlib.GROUP_EP, expert_group_members(engine.hdr, engine.rank))
    return pa
