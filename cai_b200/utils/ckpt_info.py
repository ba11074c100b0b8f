"""Print what a checkpoint file holds: step, plan hash, sections with their sizes; every section is read, so a
damaged file shows up as a checksum failure.

    python -m cai_b200.utils.ckpt_info ckpt/run [--rank 0]

The first 12 bytes keep the reference's layout (u32 step, u64 plan_hash: src/runtime.c:244-251); the section table
with per-section checksums follows.
"""
from __future__ import annotations

import argparse
import ctypes
from ctypes import c_void_p

import numpy as np

from .. import plan as planlib


def inspect(path, rank=0):
    """``{"file", "step", "plan_hash", "sections": [(name, bytes, ok)]}`` of the newest file for ``rank`` under ``path``."""
    L = planlib.lib()
    step, ph, nsec = ctypes.c_uint32(0), ctypes.c_uint64(0), ctypes.c_uint32(0)
    resolved = ctypes.create_string_buffer(1024)
    rc = L.cai_ckpt_probe(str(path).encode(), rank, ctypes.byref(step), ctypes.byref(ph), ctypes.byref(nsec), resolved, len(resolved))
    if rc != 0:
        raise IOError(f"no readable checkpoint for rank {rank} under {path}")
    sections = []
    for i in range(nsec.value):
        name = ctypes.create_string_buffer(16)
        nbytes = ctypes.c_uint64(0)
        L.cai_ckpt_section(resolved.value, i, name, ctypes.byref(nbytes), None, 0)
        buf = np.empty(nbytes.value, dtype=np.uint8)
        ok = L.cai_ckpt_section(resolved.value, i, name, ctypes.byref(nbytes), c_void_p(buf.ctypes.data), buf.nbytes) == 0
        sections.append((name.value.decode(), int(nbytes.value), ok))
    return {"file": resolved.value.decode(), "step": step.value, "plan_hash": ph.value, "sections": sections}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("path", help="checkpoint path prefix (as given to --ckpt) or a checkpoint file")
    ap.add_argument("--rank", type=int, default=0)
    a = ap.parse_args(argv)
    info = inspect(a.path, a.rank)
    print(f"{info['file']}: step {info['step']}, plan {info['plan_hash']:016x}, {len(info['sections'])} sections")
    bad = 0
    for name, n, ok in info["sections"]:
        print(f"  {name:<8} {n:>14,d} bytes  {'ok' if ok else 'CHECKSUM MISMATCH'}")
        bad += not ok
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
