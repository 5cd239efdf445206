"""Version counters of tensors that are written through raw pointers.

Kernels launched through ctypes (the optimizer's apply kernels, QK-clip, the peer
gathers) and writes through another view of a flat arena (``p.data`` is a view of the
arena, with a version counter of its own) change a parameter's values without moving
``p._version``.  Everything that keys a cache on the version counter -- the blocks'
bf16 weight copies for gradient-free passes, torch's own saved-tensor checks -- must
be told: ``mark_written`` moves the counters, without touching the data and without
a kernel launch.  (The reference updates its parameters with torch in-place ops,
reference moonlight.py ``step``, which move the counters by themselves.)
"""
from __future__ import annotations

from typing import Iterable

import torch


def mark_written(tensors: Iterable[torch.Tensor]) -> None:
    ts = [t for t in tensors if t is not None]
    if not ts:
        return
    inc = getattr(torch._C, "_increment_version", None)
    if inc is not None:
        try:
            inc(ts)
            return
        except TypeError:          # a build whose binding takes one tensor at a time
            pass
    with torch.no_grad():
        for t in ts:
            t.add_(0)              # an in-place no-op moves the counter as well
