"""Whole-matrix ownership for distributed Moonlight.

The reference repeats every Newton-Schulz on every rank
(``moonlight.py:395-437``; measured 17 % of its A100 step).  Here each Muon
matrix has ONE owner rank: gradients are reduced to the owner, the owner runs
momentum + Newton-Schulz, and the orthogonalised update is returned to all
ranks, which apply the same fp32 update so replicas stay bit-identical.

``assign_owners`` is a deterministic longest-processing-time bin packing over
the Newton-Schulz FLOP cost, so the map is a pure function of (shapes, world)
and is stable across resume; ``Trainer.save`` writes it into the checkpoint's
``extra["muon_owner"]`` and ``Trainer.load`` refuses a file whose map differs
at the same world size.
"""

from __future__ import annotations

from typing import Dict, List, Sequence, Tuple


def ns_cost(shape: Tuple[int, int], steps: int = 5) -> float:
    """FLOPs of ``steps`` iterations: Gram 2 n^2 m + A^2 2 n^3 + apply 2 n^2 m
    with n = min side."""
    n, m = min(shape), max(shape)
    return steps * (4.0 * n * n * m + 2.0 * n ** 3)


def assign_owners(shapes: Sequence[Tuple[int, int]], world: int, steps: int = 5) -> List[int]:
    """owner[i] for each matrix; ties broken by index so every rank computes
    the same map without communication."""
    order = sorted(range(len(shapes)), key=lambda i: (-ns_cost(shapes[i], steps), i))
    load = [0.0] * world
    owner = [0] * len(shapes)
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        owner[i] = r
        load[r] += ns_cost(shapes[i], steps)
    return owner


def owner_loads(shapes, owner, world, steps=5) -> List[float]:
    load = [0.0] * world
    for s, r in zip(shapes, owner):
        load[r] += ns_cost(s, steps)
    return load
