"""Device-side failure detection, on one GPU and without faulting it: a fused GEMM -> reduce-scatter is
launched as member 0 of a two-member group whose second member never runs. Its wait on that member's
arrival flags must run out (or be cut short by the host), the kernel must return with the code in the
device status word, and the context must stay usable for ordinary kernels.

The "second member" is just a second buffer on the same GPU: the kernel's peer stores land there and
nothing ever raises the flags it waits for. No kernel spins without a limit, nothing traps."""
import time
from ctypes import c_int, c_longlong, c_uint32, c_ulonglong, c_void_p

import pytest

pytestmark = pytest.mark.gpu

CAI_DEV_TIMEOUT_PEER_FLAG = 105
CAI_DEV_ABORTED_BY_HOST = 108


def _launch_with_silent_member(torch, klib, T=256, N=256, K=128):
    """Enqueue gemm_rs as rank 0 of 2; returns the tensors that must stay alive until the kernel is done."""
    L = klib.lib()
    P, I, LL, ULL = c_void_p, c_int, c_longlong, c_ulonglong
    L.cai_fused_gemm_rs_c.argtypes = [P, I, I, ULL, I, P, P, ULL, P, P, I, I, I, LL, LL, LL, LL, I, P, c_uint32, P]
    sig = int(L.cai_signal_block_bytes())
    stage_off = (sig + 1023) & ~1023
    nbytes = stage_off + T * N * 2 + 4096
    members = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    bases = (c_void_p * 2)(*[c_void_p(m.data_ptr()) for m in members])
    A = torch.randn(T, K, device="cuda").to(torch.bfloat16)
    B = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    out = torch.zeros(T // 2, N, device="cuda", dtype=torch.bfloat16)
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    st = torch.cuda.current_stream().cuda_stream
    klib.check(L.cai_fused_gemm_rs_c(bases, 0, 2, 0, 0, A.data_ptr(), B.data_ptr(), stage_off, out.data_ptr(), None, T, N, K,
                                     K, K, N, 0, 0, epoch.data_ptr(), 1, st), "gemm_rs")
    return members, A, B, out, epoch


def _ordinary_kernel_still_works(torch):
    from cai_b200.ops import gemm
    a = torch.randn(256, 128, device="cuda").to(torch.bfloat16)
    b = torch.randn(384, 128, device="cuda").to(torch.bfloat16)
    c = gemm(a, b)
    torch.cuda.synchronize()
    ref = a.float() @ b.float().t()
    assert (c.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3


def test_wait_on_a_silent_member_runs_out_and_the_context_stays_usable():
    import torch
    from cai_b200.ops import _lib as klib
    assert klib.device_status(clear=True) == 0
    klib.set_wait_limit_us(20_000)          # 20 ms instead of the default two seconds
    try:
        t0 = time.perf_counter()
        keep = _launch_with_silent_member(torch, klib)
        torch.cuda.synchronize()            # the kernel returns by itself
        waited = time.perf_counter() - t0
        assert klib.device_status(clear=False) == CAI_DEV_TIMEOUT_PEER_FLAG
        assert klib.device_status(clear=True) == CAI_DEV_TIMEOUT_PEER_FLAG   # reading does not clear unless asked
        assert klib.device_status(clear=True) == 0
        assert 0.015 < waited < 1.0, waited
        del keep
    finally:
        klib.set_wait_limit_us(0)
    _ordinary_kernel_still_works(torch)
    assert klib.device_status(clear=True) == 0


def test_host_abort_cuts_a_pending_wait_short():
    """The watchdog's lever: the host writes the abort code into the status word and the waiting kernel
    unwinds long before its own (default, ~2 s) limit."""
    import torch
    from cai_b200.ops import _lib as klib
    assert klib.device_status(clear=True) == 0
    keep = _launch_with_silent_member(torch, klib)
    time.sleep(0.05)
    t0 = time.perf_counter()
    klib.status_abort()
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert klib.device_status(clear=True) == CAI_DEV_ABORTED_BY_HOST
    del keep
    _ordinary_kernel_still_works(torch)
    assert klib.device_status(clear=True) == 0
