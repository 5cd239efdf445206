"""Learning-rate schedule (pure function of the step, so resume needs no
state): linear warm-up, then WSD (flat, then a "1-sqrt" or cosine tail over
the last ``decay_fraction`` of training) or plain cosine; floor
``lr * min_lr_ratio``.  Reference ``train.py:266-287``."""

from __future__ import annotations

import math


def lr_at(step: int, o) -> float:
    if step < o.warmup_steps:
        return o.lr * step / max(1, o.warmup_steps)
    floor = o.lr * o.min_lr_ratio
    span = o.lr - floor
    if o.lr_schedule == "wsd":
        start = int(o.total_steps * (1.0 - o.decay_fraction))
        if step < start:
            return o.lr
        x = min(1.0, (step - start) / max(1, o.total_steps - start))
        if o.decay_shape == "1-sqrt":
            return floor + span * (1.0 - math.sqrt(x))
        return floor + 0.5 * span * (1 + math.cos(math.pi * x))
    x = min(1.0, (step - o.warmup_steps) / max(1, o.total_steps - o.warmup_steps))
    return floor + 0.5 * span * (1 + math.cos(math.pi * x))
