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
