"""The fp64 oracle: finite-difference gradient checks (the reference's gate is 1e-4) and learning."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module", autouse=True)
def _built():
    from cai_b200 import _build
    _build.build_host()


def _batch(vocab, seq, B, seed=0):
    rng = np.random.default_rng(seed)
    s = rng.integers(0, vocab, size=(B, seq + 1), dtype=np.int32)
    return s[:, :-1].copy(), s[:, 1:].copy()


@pytest.mark.parametrize("kw", [
    dict(),                                             # the reference's architecture: MHA, learned positions, tied
    dict(n_kv_heads=1),                                 # grouped-query attention
    dict(rope=True),                                    # rotary embedding
    dict(rope=True, n_kv_heads=1, tied=False, init_std=0.02),
    dict(rope=True, experts=4, top_k=2),                # mixture of experts (router, top-2, renormalised weights)
    dict(n_kv_heads=1, experts=8, top_k=3, tied=False),
])
def test_backward_matches_finite_differences(kw):
    from cai_b200.models.oracle import Oracle
    o = Oracle(vocab=7, seq=4, hidden=8, layers=2, n_heads=2, head_dim=4, ffn=16, seed=3, **kw)
    tok, tgt = _batch(7, 4, 2)
    err = o.grad_check(tok, tgt, n_probe=0, h=1e-5)
    assert err < 1e-4, err


def test_adamw_halves_the_loss_on_a_fixed_batch():
    from cai_b200.models.oracle import Oracle
    o = Oracle(vocab=7, seq=4, hidden=8, layers=2, n_heads=2, head_dim=4, ffn=16, seed=5)
    tok, tgt = _batch(7, 4, 2, seed=1)
    first = o.forward(tok, tgt)
    for _ in range(300):
        o.forward(tok, tgt)
        o.backward(tok, tgt)
        o.adamw(0.01)
    assert o.forward(tok, tgt) < 0.5 * first


def test_reftrain_learns_the_shift_task():
    r = subprocess.run([str(ROOT / "bin" / "reftrain"), "--steps", "60"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout
    assert "88384 params" in r.stdout      # same parameter count as the reference's model
    assert "eval acc 100.0%" in r.stdout or "eval acc 99" in r.stdout


@pytest.mark.parametrize("experts", [0, 4])
def test_pytorch_restatement_matches_the_oracle(experts):
    """The plain PyTorch model that GPU tests compare the engine against computes the same loss and
    gradients as the finite-difference-checked fp64 oracle (GQA + RoPE, dense and mixture of experts)."""
    import torch
    from cai_b200.models.oracle import Oracle
    from cai_b200.models.reference_torch import forward_loss
    V, S, H, L, nh, nkv, hd, F, k = 11, 6, 8, 2, 2, 1, 4, 12, 2
    o = Oracle(vocab=V, seq=S, hidden=H, layers=L, n_heads=nh, n_kv_heads=nkv, head_dim=hd, ffn=F, rope=True, tied=True,
               init_std=0.3, seed=9, experts=experts, top_k=k)
    tok, tgt = _batch(V, S, 3, seed=4)
    loss = o.forward(tok, tgt)
    o.backward(tok, tgt)
    t = lambda name, *shape: torch.tensor(np.array(o.tensor(name)).reshape(shape), dtype=torch.float64)
    P = {"embed": t("E", V, H), "gf": t("gf", H)}
    for l in range(L):
        pre = f"L{l}."
        P[pre + "g1"], P[pre + "g2"] = t(pre + "g1", H), t(pre + "g2", H)
        P[pre + "wqkv"] = torch.cat([t(pre + "Wq", H, nh * hd).t(), t(pre + "Wk", H, nkv * hd).t(), t(pre + "Wv", H, nkv * hd).t()])
        P[pre + "wo"] = t(pre + "Wo", nh * hd, H).t()
        if experts:
            g, u, d = t(pre + "Wg", experts, H, F), t(pre + "Wu", experts, H, F), t(pre + "Wd", experts, F, H)
            P[pre + "wr"] = t(pre + "Wr", H, experts).t()
            P[pre + "experts.wgu"] = torch.cat([torch.cat([g[e].t(), u[e].t()]) for e in range(experts)])
            P[pre + "experts.wd"] = torch.cat([d[e].t() for e in range(experts)])
        else:
            P[pre + "wgu"] = torch.cat([t(pre + "Wg", H, F).t(), t(pre + "Wu", H, F).t()])
            P[pre + "wd"] = t(pre + "Wd", F, H).t()
    P = {n: v.contiguous().requires_grad_(True) for n, v in P.items()}
    ref = forward_loss(P, torch.tensor(tok, dtype=torch.long), torch.tensor(tgt, dtype=torch.long), layers=L, heads=nh,
                       kv_heads=nkv, head_dim=hd, seq=S, eps=1e-6, theta=10000.0, dtype=torch.float64, top_k=k)
    assert abs(ref.item() - loss) < 1e-9, (ref.item(), loss)
    ref.backward()
    g_wo = np.array(o.tensor("L1.Wo", grad=True)).reshape(nh * hd, H).T
    assert np.allclose(P["L1.wo"].grad.numpy(), g_wo, atol=1e-9)
    assert np.allclose(P["embed"].grad.numpy(), np.array(o.tensor("E", grad=True)).reshape(V, H), atol=1e-9)
    if experts:
        g_wr = np.array(o.tensor("L0.Wr", grad=True)).reshape(H, experts).T
        assert np.allclose(P["L0.wr"].grad.numpy(), g_wr, atol=1e-9)
        g_wd = np.array(o.tensor("L0.Wd", grad=True)).reshape(experts, F, H)
        assert np.allclose(P["L0.experts.wd"].grad.numpy().reshape(experts, H, F), g_wd.transpose(0, 2, 1), atol=1e-9)
