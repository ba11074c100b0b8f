"""Every fused compute+collective kernel, stand-alone, against its NCCL path: as one process with a
group of one, and over two GPUs when the box has them (cai_b200/parallel/fused_bench.py checks the
numbers itself and exits non-zero on a mismatch or a device status)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
SCRIPT = str(ROOT / "cai_b200" / "parallel" / "fused_bench.py")
CASES = {
    "ag_gemm": ["--tokens", "1024", "--out-features", "512", "--in-features", "1024"],
    "gemm_rs": ["--tokens", "1024", "--out-features", "1024", "--in-features", "512"],
    "rs_adamw": ["--params", "4194304"],
    "gather_gemm": ["--tokens", "1024", "--out-features", "1024", "--in-features", "1024"],
    "moe_exchange": ["--tokens", "512", "--in-features", "512", "--experts", "32", "--top-k", "2"],
}


def _run(op, nproc, port):
    args = ["--op", op, "--iters", "2", "--warmup", "1"] + CASES[op]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_PORT=str(port))
    if nproc == 1:
        cmd = [sys.executable, SCRIPT] + args
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
               "127.0.0.1", "--master-port", str(port), SCRIPT] + args
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-2000:])
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    res = json.loads(line)
    assert res["status"] == 0 and res["world"] == nproc and res["fused_us"] > 0
    return res


@pytest.mark.parametrize("op", sorted(CASES))
def test_fused_kernel_group_of_one(op):
    _run(op, 1, 29650 + sorted(CASES).index(op))


@pytest.mark.parametrize("op", sorted(CASES))
def test_fused_kernel_two_gpus(op):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(op, 2, 29670 + sorted(CASES).index(op))


# The shapes the headline model gives the fused tensor-parallel kernels at tp = 8 (hidden 2048, ffn 8192, 16 / 8 heads,
# 4096 tokens per microbatch, two microbatches per launch): checked against GEMM + NCCL on all eight GPUs.
TP8_SHAPES = {
    "ag_gemm": [("8192", "512", "2048"), ("8192", "2048", "2048")],      # QKV, gate/up
    "gemm_rs": [("8192", "2048", "256"), ("8192", "2048", "1024")],      # attention out, down projection
}


@pytest.mark.parametrize("op,shape", [(op, sh) for op, shapes in sorted(TP8_SHAPES.items()) for sh in shapes])
def test_fused_kernel_production_shapes_eight_gpus(op, shape):
    import torch
    if torch.cuda.device_count() < 8:
        pytest.skip("needs 8 GPUs")
    T, N, K = shape
    args = ["--op", op, "--iters", "3", "--warmup", "2", "--tokens", T, "--out-features", N, "--in-features", K]
    port = 29690 + sorted(TP8_SHAPES).index(op) * 4 + TP8_SHAPES[op].index(shape)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=8", "--master-addr", "127.0.0.1",
           "--master-port", str(port), SCRIPT] + args
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, NCCL_NVLS_ENABLE="0"), cwd=ROOT)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-2000:])
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert res["status"] == 0 and res["world"] == 8
