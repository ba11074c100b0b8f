"""Flash attention (forward and backward) against a plain PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_attention(qkv, B, S, nh, nkv, hd):
    x = qkv.float().view(B, S, nh + 2 * nkv, hd)
    q = x[:, :, :nh].transpose(1, 2)                       # B nh S hd
    k = x[:, :, nh:nh + nkv].transpose(1, 2)
    v = x[:, :, nh + nkv:].transpose(1, 2)
    rep = nh // nkv
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    s = (q @ k.transpose(-1, -2)) * hd ** -0.5
    mask = torch.ones(S, S, device=qkv.device, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.softmax(s, -1) @ v
    return o.transpose(1, 2).reshape(B * S, nh * hd), lse


@pytest.mark.parametrize("B,S,nh,nkv", [(1, 128, 2, 2), (2, 256, 4, 2), (1, 384, 4, 1), (1, 1024, 8, 2),
                                        (2, 2048, 4, 4), (1, 4096, 16, 8)])
@pytest.mark.parametrize("variant", [1, 2])
def test_flash_attn_fwd(B, S, nh, nkv, variant):
    from cai_b200 import ops
    torch.manual_seed(0)
    hd = 128
    qkv = torch.randn(B * S, (nh + 2 * nkv) * hd, device="cuda").to(torch.bfloat16)
    out, lse = ops.flash_attn_fwd(qkv, B, S, nh, nkv, hd, variant=variant)
    ref, lse_ref = _ref_attention(qkv, B, S, nh, nkv, hd)
    rel = ((out.float() - ref).norm() / ref.norm()).item()
    assert rel < 1e-2, rel
    assert (out.float() - ref).abs().max().item() < 6e-2
    assert torch.allclose(lse, lse_ref, atol=2e-2, rtol=1e-3)


# The dK / dV kernel has two forms: one CTA per kv group looping over the group's query heads (grids that fill
# the GPU: B * kv groups * key tiles >= SM count) and one CTA per query head with chained adds (small grids).
# (1, 4096, 16, 8) is the shape of the headline model on one GPU and takes the first form with two heads per
# group; (1, 512, 8, 1) chains eight heads; (2, 4096, 2, 1) is the tp = 8 shape with two microbatches per launch.
@pytest.mark.parametrize("B,S,nh,nkv", [(1, 128, 2, 2), (2, 256, 4, 2), (1, 384, 4, 1), (1, 1024, 8, 2),
                                        (1, 4096, 16, 8), (1, 512, 8, 1), (2, 4096, 2, 1)])
def test_flash_attn_bwd(B, S, nh, nkv):
    from cai_b200 import ops
    if not hasattr(ops.lib(), "cai_flash_attn_bwd"):
        pytest.skip("backward kernel not built")
    torch.manual_seed(1)
    hd = 128
    qkv = torch.randn(B * S, (nh + 2 * nkv) * hd, device="cuda").to(torch.bfloat16)
    dout = torch.randn(B * S, nh * hd, device="cuda").to(torch.bfloat16)
    out, lse = ops.flash_attn_fwd(qkv, B, S, nh, nkv, hd)
    dqkv = ops.flash_attn_bwd(qkv, out, dout, lse, B, S, nh, nkv, hd)
    x = qkv.float().requires_grad_(True)
    ref, _ = _ref_attention(x, B, S, nh, nkv, hd)
    ref.backward(dout.float())
    g = x.grad.view(B * S, nh + 2 * nkv, hd)
    d = dqkv.float().view(B * S, nh + 2 * nkv, hd)
    for name, sl in (("dq", slice(0, nh)), ("dk", slice(nh, nh + nkv)), ("dv", slice(nh + nkv, nh + 2 * nkv))):
        rel = ((d[:, sl] - g[:, sl]).norm() / g[:, sl].norm()).item()
        assert rel < 2e-2, (name, rel)
