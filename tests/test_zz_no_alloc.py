"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some callers of the kernel library cannot allocate device memory where they call it (under a
fixed start-up memory budget, in a latency-bound loop that must not enter an allocator, from a
plug-in that must not touch the host's allocator). ``cai_rmsnorm_bwd_static`` serves them: its scratch is a fixed array inside the
library. This test checks it against the regular entry point, twice in a row (the array is shared
between calls and keeps old contents, so the second call must not be disturbed by the first), and
checks that sizes beyond the fixed maximum are refused. It sits last in collection order so that
a failure here cannot hide other results in a run that stops at the first failure.
"""
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _fn():
    from cai_b200.ops import _lib
    L = _lib.lib()
    f = L.cai_rmsnorm_bwd_static
    f.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    f.restype = c_int
    return L, f


def _case(rows, H, seed):
    torch.manual_seed(seed)
    x = torch.randn(rows, H, device="cuda").to(torch.bfloat16)
    g = (1.0 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
    dy = torch.randn(rows, H, device="cuda").to(torch.bfloat16)
    return x, g, dy


def test_static_entry_point_matches_regular_one_twice_in_a_row():
    from cai_b200 import ops
    L, f = _fn()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second reuses the array the first one dirtied
    for rows, H, seed in ((700, 2048, 0), (333, 4096, 1)):
        x, g, dy = _case(rows, H, seed)
        _, rstd = ops.rmsnorm_fwd(x, g, 1e-6)
        base = torch.randn(rows, H, device="cuda").to(torch.bfloat16)
        dx_ref, dg_ref = base.clone(), torch.ones(H, device="cuda")
        ops.rmsnorm_bwd(x, g, rstd, dy, dx=dx_ref, dg=dg_ref, dx_accumulate=True, dg_accumulate=True)
        dx, dg = base.clone(), torch.ones(H, device="cuda")
        rc = f(x.data_ptr(), g.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dx.data_ptr(), dg.data_ptr(), rows, H, 1, 1,
               stream)
        assert rc == 0, L.cai_last_error()
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref)                       # per-row math is the same kernel
        assert ((dg - dg_ref).norm() / dg_ref.norm()).item() < 1e-3
        # and against plain PyTorch fp32
        xf = x.float().requires_grad_(True)
        gf = g.float().requires_grad_(True)
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * gf
        y.backward(dy.float())
        assert ((dg - (1.0 + gf.grad)).norm() / gf.grad.norm()).item() < 1e-3
        assert ((dx.float() - (base.float() + xf.grad)).norm() / xf.grad.norm()).item() < 2e-2


def test_static_entry_point_rejects_rows_wider_than_its_array():
    L, f = _fn()
    x, g, dy = _case(8, 8192, 2)
    rstd = torch.ones(8, device="cuda")
    dx = torch.empty_like(x)
    dg = torch.zeros(8192, device="cuda")
    rc = f(x.data_ptr(), g.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dx.data_ptr(), dg.data_ptr(), 8, 8192, 0, 0,
           torch.cuda.current_stream().cuda_stream)
    assert rc < 0 and b"at most 4096" in L.cai_last_error()
