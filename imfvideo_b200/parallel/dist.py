"""Process-group plumbing: one process per GPU, NCCL over NVLink on CUDA,
gloo on CPU (reference ``train.py:84-100``, ``:377-389``).  Adds what the
reference lacks: an initial weight broadcast (it seeds each rank differently
and never synchronises, ``train.py:391-396``), a bounded collective timeout,
and a host-side heartbeat so a missing rank is noticed before the next launch.
"""

from __future__ import annotations

import datetime
import os
import threading
import time
from typing import Iterable, Optional, Tuple

import torch
import torch.distributed as dist


def resolve_device() -> Tuple[torch.device, str]:
    if torch.cuda.is_available():
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
        return torch.device("cuda"), "nccl"
    return torch.device("cpu"), "gloo"


def init_distributed(timeout_s: float = 600.0) -> Tuple[int, int, int, torch.device]:
    """Returns (rank, world, local_rank, device).  Single process when
    WORLD_SIZE is unset or 1."""
    device, backend = resolve_device()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        if device.type == "cuda":
            torch.cuda.set_device(0)
            device = torch.device("cuda", 0)
        return 0, 1, 0, device
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if device.type == "cuda":
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    kw = dict(backend=backend, timeout=datetime.timedelta(seconds=timeout_s))
    if device.type == "cuda":
        kw["device_id"] = device
    dist.init_process_group(**kw)
    return dist.get_rank(), dist.get_world_size(), local_rank, device


def is_dist() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def world_size() -> int:
    return dist.get_world_size() if is_dist() else 1


def get_rank() -> int:
    return dist.get_rank() if is_dist() else 0


def barrier() -> None:
    if is_dist():
        dist.barrier()


@torch.no_grad()
def broadcast_module(module: torch.nn.Module, src: int = 0) -> None:
    """Make every replica start from rank ``src``'s parameters and buffers
    (one flat broadcast per dtype)."""
    if not is_dist():
        return
    by_dtype = {}
    for t in list(module.parameters()) + list(module.buffers()):
        by_dtype.setdefault((t.dtype, t.device), []).append(t)
    for ts in by_dtype.values():
        flat = torch.cat([t.detach().reshape(-1) for t in ts])
        dist.broadcast(flat, src=src)
        off = 0
        for t in ts:
            n = t.numel()
            t.copy_(flat[off:off + n].view_as(t))
            off += n


def all_reduce_max_(t: torch.Tensor) -> torch.Tensor:
    if is_dist():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t


def shutdown() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


class Heartbeat:
    """Host-side liveness: each rank bumps ``hb/{rank}`` in the process
    group's store from a daemon thread; ``check()`` (called between steps,
    never with a collective in flight) raises ``RankLostError`` naming ranks
    whose counter has not moved for ``stale_s`` seconds.  Nothing here touches
    the GPU, so a lost rank is detected without a hung collective."""

    def __init__(self, store, rank: int, world: int, period_s: float = 1.0,
                 stale_s: float = 10.0):
        self.store, self.rank, self.world = store, rank, world
        self.period_s, self.stale_s = period_s, stale_s
        self._stop = threading.Event()
        self._seen = {r: (-1, time.monotonic()) for r in range(world)}
        self._thread = threading.Thread(target=self._beat, daemon=True)

    def start(self) -> "Heartbeat":
        self.store.add(f"hb/{self.rank}", 1)
        self._thread.start()
        return self

    def _beat(self) -> None:
        while not self._stop.wait(self.period_s):
            try:
                self.store.add(f"hb/{self.rank}", 1)
            except Exception:
                return

    def check(self) -> None:
        now = time.monotonic()
        lost = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = int(self.store.add(f"hb/{r}", 0))
            except Exception:
                val = self._seen[r][0]
            last, when = self._seen[r]
            if val != last:
                self._seen[r] = (val, now)
            elif now - when > self.stale_s:
                lost.append(r)
        if lost:
            raise RankLostError(lost)

    def stop(self) -> None:
        self._stop.set()


class RankLostError(RuntimeError):
    def __init__(self, ranks: Iterable[int]):
        self.ranks = list(ranks)
        super().__init__(f"no heartbeat from rank(s) {self.ranks}")
