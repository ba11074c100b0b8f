"""Learning-rate schedule of the device trainer (host arithmetic)."""
import math

import pytest


def test_warmup_then_constant():
    from cai_b200.utils.schedule import lr_at
    assert [round(lr_at(s, 1e-3, warmup=4), 7) for s in range(6)] == [0.00025, 0.0005, 0.00075, 0.001, 0.001, 0.001]
    assert lr_at(0, 3e-4) == 3e-4 and lr_at(10 ** 6, 3e-4) == 3e-4


@pytest.mark.parametrize("decay", ["cosine", "linear"])
def test_decay_reaches_the_floor_at_the_last_step_and_stays(decay):
    from cai_b200.utils.schedule import lr_at
    base, warm, total = 2e-3, 10, 110
    rates = [lr_at(s, base, warm, total, decay, 0.1) for s in range(130)]
    assert rates[warm - 1] == pytest.approx(base) and rates[warm] == pytest.approx(base)
    assert all(a >= b - 1e-15 for a, b in zip(rates[warm:], rates[warm + 1:]))          # never rises after the warm-up
    assert rates[total - 1] == pytest.approx(0.1 * base) and rates[-1] == pytest.approx(0.1 * base)
    mid = rates[warm + (total - 1 - warm) // 2]
    assert mid == pytest.approx(base * (0.1 + 0.9 * (0.5 if decay == "linear" else 0.5 * (1 + math.cos(math.pi * 0.5)))), rel=0.03)


def test_unknown_decay_is_an_error():
    from cai_b200.utils.schedule import lr_at
    with pytest.raises(ValueError):
        lr_at(50, 1e-3, 0, 100, "exponential")
