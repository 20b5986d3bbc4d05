"""Learning-rate multipliers, stepped once per optimizer step.

WSD = linear warm-up, flat, cosine to zero over the last ``decay_ratio`` of the
run; cosine = warm-up then cosine to ``min_lr_ratio``
(reference: train/utils.py:529-576).  The multipliers are plain functions of
the step so they can be unit-tested and re-created after a resume; they are
wrapped in ``torch.optim.lr_scheduler.LambdaLR`` so the checkpoint keeps the
same ``scheduler`` entry the reference writes.
"""
from __future__ import annotations

import math
from typing import Callable


def wsd_multiplier(total_steps: int, warmup_steps: int, decay_ratio: float) -> Callable[[int], float]:
    decay = int(decay_ratio * total_steps)
    stable = total_steps - warmup_steps - decay

    def f(step: int) -> float:
        if step < warmup_steps:
            return step / max(1, warmup_steps)
        if step < warmup_steps + stable:
            return 1.0
        t = min(1.0, (step - warmup_steps - stable) / max(1, decay))
        return 0.5 * (1.0 + math.cos(math.pi * t))

    return f


def cosine_multiplier(total_steps: int, warmup_steps: int, min_lr_ratio: float) -> Callable[[int], float]:
    def f(step: int) -> float:
        if step < warmup_steps:
            return step / max(1, warmup_steps)
        t = min(1.0, (step - warmup_steps) / max(1, total_steps - warmup_steps))
        return min_lr_ratio + (1.0 - min_lr_ratio) * 0.5 * (1.0 + math.cos(math.pi * t))

    return f


def make_multiplier(kind: str, total_steps: int, warmup_steps: int, *, wsd_decay_ratio: float = 0.1,
                    min_lr_ratio: float = 0.1) -> Callable[[int], float]:
    if kind == "wsd":
        return wsd_multiplier(total_steps, warmup_steps, wsd_decay_ratio)
    if kind == "cosine":
        return cosine_multiplier(total_steps, warmup_steps, min_lr_ratio)
    raise ValueError(f"unknown scheduler_type {kind!r} (expected 'wsd' or 'cosine')")


def build_scheduler(optimizer, kind: str, total_steps: int, warmup_steps: int, **kw):
    from torch.optim.lr_scheduler import LambdaLR

    return LambdaLR(optimizer, make_multiplier(kind, total_steps, warmup_steps, **kw))


def accumulation_pattern(multiplier: float, max_len: int = 100) -> list[int]:
    """Integer micro-batch counts whose mean is ``multiplier`` (≥ 1), cycled by
    the trainer: 1.5 → [1, 2], 2.0 → [2]  (reference: train/utils.py:88-104)."""
    if multiplier < 1.0:
        raise ValueError("tpi_multiplier must be >= 1")
    out = []
    for i in range(max_len):
        hi = (i + 1) * multiplier
        out.append(int(math.floor(hi + 1e-9)) - int(math.floor(i * multiplier + 1e-9)))
        if abs(hi - round(hi)) < 1e-9:
            break
    return out
