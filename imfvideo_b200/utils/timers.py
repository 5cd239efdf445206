"""Phase timers and NVTX ranges (the reference has neither; its step
breakdowns came from uncommitted scripts).  ``PhaseTimer`` brackets named
phases with CUDA events on the current stream; ``summary`` synchronises once
and returns milliseconds per phase; ``reduce_max`` takes the max over ranks,
which is how every multi-GPU number in this repo is reported."""

from __future__ import annotations

import contextlib
import time
from collections import defaultdict
from typing import Dict, List, Tuple

import torch


class PhaseTimer:
    def __init__(self, enabled: bool = True, nvtx: bool = True):
        self.enabled = enabled
        self.cuda = torch.cuda.is_available()
        self.nvtx = nvtx and self.cuda
        self._pairs: Dict[str, List[Tuple]] = defaultdict(list)
        self._cpu: Dict[str, float] = defaultdict(float)

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                yield
            finally:
                b.record()
                self._pairs[name].append((a, b))
                if self.nvtx:
                    torch.cuda.nvtx.range_pop()
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._cpu[name] += (time.perf_counter() - t0) * 1e3

    def summary(self, reset: bool = True) -> Dict[str, float]:
        out = dict(self._cpu)
        if self.cuda and self._pairs:
            torch.cuda.synchronize()
            for name, pairs in self._pairs.items():
                out[name] = out.get(name, 0.0) + sum(a.elapsed_time(b) for a, b in pairs)
        if reset:
            self._pairs.clear()
            self._cpu.clear()
        return out

    @staticmethod
    def reduce_max(ms: Dict[str, float]) -> Dict[str, float]:
        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
            return ms
        keys = sorted(ms)
        dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
        t = torch.tensor([ms[k] for k in keys], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return dict(zip(keys, t.tolist()))
