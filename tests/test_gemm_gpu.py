"""tcgen05 GEMM against a plain PyTorch fp32 reference, all operand layouts and epilogues."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, ta, tb):
    A = a.float().t() if ta else a.float()
    B = b.float() if tb else b.float().t()
    return A @ B


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (300, 264, 200), (1024, 2048, 1024),
                                     (4096, 1024, 512), (77, 136, 1000)])
def test_gemm_layouts(M, N, K, ta, tb):
    from cai_b200 import ops
    torch.manual_seed(0)
    if ta and M % 8:
        M = (M + 7) // 8 * 8
    if K % 8:
        K = (K + 7) // 8 * 8
    a = torch.randn((K, M) if ta else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if tb else (N, K), device="cuda", dtype=torch.bfloat16)
    c = ops.gemm(a, b, trans_a=ta, trans_b=tb, out_dtype=torch.float32)
    ref = _ref(a, b, ta, tb)
    err = (c - ref).abs().max().item()
    assert err <= 2e-3 * (K ** 0.5) + 1e-3, f"max err {err}"
    cb = ops.gemm(a, b, trans_a=ta, trans_b=tb)
    assert cb.dtype == torch.bfloat16
    rel = ((cb.float() - ref).norm() / ref.norm()).item()
    assert rel < 5e-3, rel


def test_gemm_epilogues():
    from cai_b200 import ops
    torch.manual_seed(1)
    M, N, K = 512, 384, 320
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    acc = torch.full((M, N), 3.0, device="cuda", dtype=torch.float32)
    ops.gemm(a, b, out=acc, accumulate=True, alpha=0.5)
    assert torch.allclose(acc, 3.0 + 0.5 * ref, atol=2e-2, rtol=1e-3)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    out = ops.gemm(a, b, residual=res)
    want = (ref + res.float())
    assert ((out.float() - want).norm() / want.norm()).item() < 5e-3
    # residual aliasing the output (h += x @ w^T)
    h = res.clone()
    ops.gemm(a, b, out=h, residual=h)
    assert torch.equal(h, out)


def test_gemm_many_tiles_persistent():
    """More tiles than SMs, so each CTA walks several tiles and both accumulators get reused."""
    from cai_b200 import ops
    torch.manual_seed(2)
    M, N, K = 4096, 4096, 256
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c = ops.gemm(a, b, out_dtype=torch.float32)
    ref = a.float() @ b.float().t()
    assert (c - ref).abs().max().item() < 0.1
    c2 = ops.gemm(a, b, out_dtype=torch.float32, sm_limit=16)
    assert torch.equal(c, c2)


@pytest.mark.parametrize("M,F,K", [(256, 128, 128), (1024, 1024, 512), (300, 384, 264), (4096, 4096, 256)])
def test_gemm_with_swiglu_in_the_epilogue(M, F, K):
    """gate/up projection + SwiGLU in one kernel, and the down projection's input gradient + SwiGLU backward in
    one kernel, against the fp32 formulas applied to the same bf16-rounded intermediates."""
    from cai_b200 import ops
    torch.manual_seed(3)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    wgu = (torch.randn(2 * F, K, device="cuda") * K ** -0.5).to(torch.bfloat16)
    gu, act = ops.gemm_swiglu(x, wgu)
    ref_gu = x.float() @ wgu.float().t()
    assert ((gu.float() - ref_gu).norm() / ref_gu.norm()).item() < 5e-3
    g, u = gu[:, :F].float(), gu[:, F:].float()
    ref_act = torch.nn.functional.silu(g) * u
    assert (act.float() - ref_act).abs().max().item() <= 1e-2 * ref_act.abs().max().item() + 1e-3
    assert torch.equal(act, ops.swiglu_fwd(gu))           # same numbers as the stand-alone kernel
    # backward: dgu = [dact * up * silu'(gate) | dact * silu(gate)] with dact = dy @ wd
    H = K
    dy = torch.randn(M, H, device="cuda", dtype=torch.bfloat16)
    wd = (torch.randn(H, F, device="cuda") * H ** -0.5).to(torch.bfloat16)
    dgu = ops.gemm_swiglu_bwd(dy, wd, gu)
    dact = ops.gemm(dy, wd, trans_b=True)
    want = ops.swiglu_bwd(gu, dact)
    assert (dgu.float() - want.float()).abs().max().item() <= 2e-2 * want.float().abs().max().item() + 1e-3
    s = torch.sigmoid(g)
    d = dy.float() @ wd.float()
    ref = torch.cat([d * u * s * (1 + g * (1 - s)), d * g * s], dim=1)
    assert ((dgu.float() - ref).norm() / ref.norm()).item() < 1e-2
