"""Gradient synchronisation strategies behind one interface.

``FlatAllReduce`` is the reference's scheme (one flat fp32 all-reduce after
the whole backward, ``train.py:353-371``) and serves as the baseline arm.
The NVLink-native path (reduce-scatter of the flat gradient arena to the Muon
owners and AdamW shards over peer memory, owner-partitioned Moonlight, update
all-gather fused into the weight update) lives in ``parallel/flat_engine.py``
and ``ops/comm_impl.py``.
"""

from __future__ import annotations

from typing import Iterable, List

import torch
import torch.distributed as dist


class GradSync:
    """Interface: ``sync()`` leaves the mean gradient in every ``p.grad``."""

    def sync(self) -> None:  # pragma: no cover - interface
        raise NotImplementedError


class NoSync(GradSync):
    def sync(self) -> None:
        return


class FlatAllReduce(GradSync):
    def __init__(self, params: Iterable[torch.nn.Parameter], world: int):
        self.params: List[torch.nn.Parameter] = list(params)
        self.world = world

    @torch.no_grad()
    def sync(self) -> None:
        grads = [p.grad for p in self.params if p.grad is not None]
        if not grads or self.world == 1:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM)
        flat.div_(self.world)
        off = 0
        for g in grads:
            n = g.numel()
            g.copy_(flat[off:off + n].view_as(g))
            off += n


def all_reduce_grads(params, world: int) -> None:
    """Function form kept for reference-API parity (``train.py:353``)."""
    FlatAllReduce(list(params), world).sync()
