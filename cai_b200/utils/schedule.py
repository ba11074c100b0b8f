"""Learning-rate schedule of the device trainer: linear warm-up, then constant, cosine or linear decay.

The plan carries the base rate (`lr` in the configuration); the executor takes the rate of every step as a parameter
(it travels with the step's other scalars), so the schedule is host arithmetic and costs nothing on the device. The
reference trains at a constant rate (tools/reftrain.c, tools/gpu_trainer.c).
"""
from __future__ import annotations

import math


def lr_at(step: int, base: float, warmup: int = 0, total: int = 0, decay: str = "none", min_ratio: float = 0.1) -> float:
    """Rate of the optimizer step with 0-based index ``step``.

    ``warmup`` steps rise linearly from ``base / warmup`` to ``base``; afterwards ``decay`` ("none", "cosine", "linear")
    takes the rate to ``min_ratio * base`` at step ``total - 1`` and keeps it there."""
    if warmup > 0 and step < warmup:
        return base * (step + 1) / warmup
    if decay == "none" or total <= warmup + 1:
        return base
    t = min(1.0, (step - warmup) / max(1, total - 1 - warmup))
    if decay == "cosine":
        f = 0.5 * (1.0 + math.cos(math.pi * t))
    elif decay == "linear":
        f = 1.0 - t
    else:
        raise ValueError(f"unknown decay '{decay}'")
    return base * (min_ratio + (1.0 - min_ratio) * f)
