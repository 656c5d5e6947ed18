"""Learning-rate schedules (iteration-indexed) and the Muon momentum warm-up.

Closed forms follow training/optimizer.py:115-187 and training/trainer.py:478-481 of the reference.
"""

from __future__ import annotations

import math
from bisect import bisect


def get_cosine_lr(t: int, lr_max: float, lr_min: float, warmup_steps: int, cosine_steps: int) -> float:
    """Linear warm-up from 0, half-cosine from lr_max to lr_min until ``cosine_steps``, then lr_min."""
    if t < warmup_steps:
        return t / warmup_steps * lr_max
    if t < cosine_steps:
        frac = (t - warmup_steps) / (cosine_steps - warmup_steps)
        return lr_min + 0.5 * (1.0 + math.cos(frac * math.pi)) * (lr_max - lr_min)
    return lr_min


def get_wsd_lr(
    t: int,
    lr_max: float,
    lr_min: float,
    zero_lr_steps: int,
    warmup_steps: int,
    decay_steps: int,
    start_decay_step: int,
    need_warmup: bool = True,
    wsd_phase: str = "stable",
) -> float:
    """Warm-up / stable / decay.

    stable phase: ``zero_lr_steps`` iterations at 0 (for model surgery), then a linear warm-up over
    ``warmup_steps``, then ``lr_max``.  decay phase: ``lr_min + (1 - sqrt(progress)) (lr_max - lr_min)``
    with progress measured from ``start_decay_step`` over ``decay_steps``.
    """
    if wsd_phase == "stable":
        if need_warmup and t < zero_lr_steps + warmup_steps:
            if t < zero_lr_steps:
                return 0.0
            return (t - zero_lr_steps) / warmup_steps * lr_max
        return lr_max
    progress = (t - start_decay_step) / decay_steps
    return lr_min + (1.0 - math.sqrt(max(progress, 0.0))) * (lr_max - lr_min)


def get_seesaw_lr(t: int, lr_max: float, warmup_steps: int, seesaw_steps) -> float:
    """Step schedule: after the k-th boundary the rate is lr_max * 2^(-k/2) (the trainer doubles the
    gradient-accumulation factor at the same boundaries)."""
    if t < warmup_steps:
        return t / warmup_steps * lr_max
    seesaw_steps = list(seesaw_steps)
    if not seesaw_steps or t < seesaw_steps[0]:
        return lr_max
    return lr_max * 2.0 ** (-bisect(seesaw_steps, t) / 2)


def muon_momentum_warmup(iteration: int, momentum: float, start: float = 0.85, steps: int = 300) -> float:
    """Momentum ramps linearly from ``start`` to ``momentum`` over the first ``steps`` iterations."""
    if iteration >= steps:
        return momentum
    return start + min(max(iteration, 1), steps) / steps * (momentum - start)
