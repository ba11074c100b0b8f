"""Bandwidth-bound kernels against plain PyTorch fp32 references."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(x):
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("rows,H", [(37, 256), (512, 2048), (100, 4096), (8192, 2048), (3000, 1024), (64, 6144)])
def test_rmsnorm_fwd_bwd(rows, H):
    from cai_b200 import ops
    torch.manual_seed(0)
    x = _bf(torch.randn(rows, H, device="cuda"))
    g = _bf(1.0 + 0.1 * torch.randn(H, device="cuda"))
    dy = _bf(torch.randn(rows, H, device="cuda"))
    y, rstd = ops.rmsnorm_fwd(x, g, 1e-6)
    xf = x.float().requires_grad_(True)
    gf = g.float().requires_grad_(True)
    rr = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)
    yr = xf * rr * gf
    assert torch.allclose(y.float(), yr, atol=2e-2, rtol=2e-2)
    assert torch.allclose(rstd, rr.squeeze(-1), rtol=1e-4)
    yr.backward(dy.float())
    dx, dg = ops.rmsnorm_bwd(x, g, rstd, dy)
    assert ((dx.float() - xf.grad).norm() / xf.grad.norm()).item() < 1e-2
    assert ((dg - gf.grad).norm() / gf.grad.norm()).item() < 1e-3
    # accumulate forms
    base = _bf(torch.randn(rows, H, device="cuda"))
    dx2 = base.clone()
    dg2 = torch.ones(H, device="cuda")
    ops.rmsnorm_bwd(x, g, rstd, dy, dx=dx2, dg=dg2, dx_accumulate=True, dg_accumulate=True)
    assert ((dx2.float() - (base.float() + xf.grad)).norm() / xf.grad.norm()).item() < 2e-2
    assert ((dg2 - (1.0 + gf.grad)).norm() / gf.grad.norm()).item() < 1e-3


def _rope_ref(x, seq, hd, theta, inverse=False):
    # x: [T, heads, hd] float
    T = x.shape[0]
    half = hd // 2
    pos = (torch.arange(T, device=x.device) % seq).float()
    inv = theta ** (-torch.arange(half, device=x.device).float() / half)
    ang = pos[:, None] * inv[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    if inverse:
        s = -s
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


def test_rope_roundtrip_and_reference():
    from cai_b200 import ops
    torch.manual_seed(0)
    T, seq, nh, nkv, hd = 96, 48, 4, 2, 128
    qkv = _bf(torch.randn(T, (nh + 2 * nkv) * hd, device="cuda"))
    orig = qkv.clone()
    table = ops.rope_table(seq, hd, 10000.0)
    ops.rope_apply_(qkv, table, seq, nh, nkv, hd)
    ref = orig.float().view(T, nh + 2 * nkv, hd).clone()
    ref[:, : nh + nkv] = _rope_ref(ref[:, : nh + nkv], seq, hd, 10000.0)
    assert torch.allclose(qkv.float().view(T, -1, hd), ref, atol=3e-2, rtol=2e-2)
    # v heads untouched
    assert torch.equal(qkv.view(T, -1, hd)[:, nh + nkv:], orig.view(T, -1, hd)[:, nh + nkv:])
    ops.rope_apply_(qkv, table, seq, nh, nkv, hd, inverse=True)
    assert torch.allclose(qkv.float(), orig.float(), atol=5e-2, rtol=3e-2)


def test_swiglu():
    from cai_b200 import ops
    torch.manual_seed(0)
    T, F = 200, 512
    gu = _bf(torch.randn(T, 2 * F, device="cuda"))
    dact = _bf(torch.randn(T, F, device="cuda"))
    act = ops.swiglu_fwd(gu)
    guf = gu.float().requires_grad_(True)
    ref = torch.nn.functional.silu(guf[:, :F]) * guf[:, F:]
    assert torch.allclose(act.float(), ref, atol=2e-2, rtol=2e-2)
    ref.backward(dact.float())
    dgu = ops.swiglu_bwd(gu, dact)
    assert ((dgu.float() - guf.grad).norm() / guf.grad.norm()).item() < 1e-2


def test_embedding():
    from cai_b200 import ops
    torch.manual_seed(0)
    V, H, T = 1000, 256, 333
    E = _bf(torch.randn(V, H, device="cuda"))
    tok = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
    out = ops.embed_fwd(tok, E)
    assert torch.equal(out, E[tok.long()])
    dout = _bf(torch.randn(T, H, device="cuda"))
    dE = torch.zeros(V, H, device="cuda")
    ops.embed_bwd_(tok, dout, dE)
    ref = torch.zeros(V, H, device="cuda").index_add_(0, tok.long(), dout.float())
    assert torch.allclose(dE, ref, atol=1e-4)
    # many tokens per row, a vocabulary that is not a multiple of the rows a CTA owns, a slice, and the same bits twice
    V2, T2 = 77, 5000
    tok2 = torch.randint(0, V2, (T2,), device="cuda", dtype=torch.int32)
    d2 = _bf(torch.randn(T2, H, device="cuda"))
    a = ops.embed_bwd_(tok2, d2, torch.zeros(V2, H, device="cuda"))
    b = ops.embed_bwd_(tok2, d2, torch.zeros(V2, H, device="cuda"))
    assert torch.equal(a, b)
    ref2 = torch.zeros(V2, H, device="cuda").index_add_(0, tok2.long(), d2.float())
    assert torch.allclose(a, ref2, atol=2e-3, rtol=1e-4)
    part = ops.embed_bwd_(tok2, d2, torch.zeros(30, H, device="cuda"), vocab_lo=20, vocab_hi=50)
    assert torch.allclose(part, ref2[20:50], atol=2e-3, rtol=1e-4)
    # vocabulary slice [250, 500)
    out2 = ops.embed_fwd(tok, E[250:500].contiguous(), vocab_lo=250, vocab_hi=500)
    mask = ((tok >= 250) & (tok < 500))
    assert torch.equal(out2[mask], E[tok.long()][mask])
    assert out2[~mask].abs().sum().item() == 0


@pytest.mark.parametrize("rows,V", [(64, 256), (200, 32000), (16, 128256)])
def test_cross_entropy(rows, V):
    from cai_b200 import ops
    torch.manual_seed(0)
    logits = _bf(3.0 * torch.randn(rows, V, device="cuda"))
    tgt = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    tgt[3] = -1
    lf = logits.float().requires_grad_(True)
    valid = tgt >= 0
    loss_ref = torch.nn.functional.cross_entropy(lf[valid], tgt[valid].long(), reduction="sum") / rows
    loss_ref.backward()
    loss = torch.zeros(1, device="cuda")
    lse = torch.empty(rows, device="cuda")
    ops.cross_entropy_(logits, tgt, loss, grad_scale=1.0 / rows, loss_scale=1.0 / rows, row_lse=lse)
    assert abs(loss.item() - loss_ref.item()) < 2e-3 * max(1.0, abs(loss_ref.item()))
    assert torch.allclose(lse, torch.logsumexp(lf.detach(), -1), atol=1e-3, rtol=1e-4)
    g = logits.float()
    assert ((g - lf.grad).norm() / lf.grad.norm()).item() < 1e-2
    assert g[3].abs().sum().item() == 0


def test_adamw_matches_reference_rule():
    from cai_b200 import ops
    torch.manual_seed(0)
    n = 10007
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr, mr, vr = p.double().clone(), m.double().clone(), v.double().clone()
    lr, b1, b2, eps, wd = 1e-3, 0.9, 0.999, 1e-8, 0.01
    for step in range(1, 4):
        ops.adamw_(p, m, v, g, pb, step, lr, b1, b2, eps, wd, grad_scale=0.5)
        gd = g.double() * 0.5
        mr = b1 * mr + (1 - b1) * gd
        vr = b2 * vr + (1 - b2) * gd * gd
        mh, vh = mr / (1 - b1 ** step), vr / (1 - b2 ** step)
        pr = pr - lr * (mh / (vh.sqrt() + eps) + wd * pr)
    assert torch.allclose(p.double(), pr, atol=1e-5, rtol=1e-5)
    assert torch.equal(pb, p.to(torch.bfloat16))
