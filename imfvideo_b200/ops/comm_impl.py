"""Peer-memory plumbing for ``csrc/comm.cu``: symmetric allocations (torch's
symmetric-memory allocator supplies the peer-mapped pointers), epoch counter,
and the launch wrappers.  Every rank must call the same methods in the same
order (each call consumes one barrier epoch)."""

from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from . import kernels as K

_lib = K._lib
vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_long

if K._has("imf_comm_reduce"):
    _lib.imf_comm_reduce.restype = ci
    _lib.imf_comm_reduce.argtypes = [vp, vp, vp, ci, ci, cl, cl, cl, ci, vp, vp, vp, vp, vp]
    _lib.imf_comm_gather.restype = ci
    _lib.imf_comm_gather.argtypes = [vp, vp, ci, ci, cl, cl, ci, ci, vp, vp]
    _lib.imf_comm_barrier.restype = ci
    _lib.imf_comm_barrier.argtypes = [vp, vp, ci, ci, ci, vp, vp]
    _lib.imf_comm_muon_apply.restype = ci
    _lib.imf_comm_muon_apply.argtypes = [vp, vp, ci, ci, cl, vp, vp, vp, ci, cl, ctypes.c_float, vp,
                                         ci, ci, vp, vp]
    _lib.imf_comm_set_wait_ns.restype = ctypes.c_ulonglong
    _lib.imf_comm_set_wait_ns.argtypes = [ctypes.c_ulonglong]


def set_peer_wait(seconds: float) -> float:
    """Bound of every later device-side wait on a peer's flag; returns the previous bound."""
    return _lib.imf_comm_set_wait_ns(int(max(1e-6, seconds) * 1e9)) / 1e9


def _ptr_array(ptrs: List[int]):
    return (vp * len(ptrs))(*[vp(int(p)) for p in ptrs])


class PeerComm:
    MAX_RANKS = 16

    def __init__(self, world: int, rank: int, device: torch.device, total: int, seg_pad: int):
        if not K._has("imf_comm_reduce"):
            raise RuntimeError("kernel library has no comm kernels")
        if world > self.MAX_RANKS:
            raise RuntimeError(f"at most {self.MAX_RANKS} ranks")
        import torch.distributed._symmetric_memory as symm

        self.world, self.rank, self.device = world, rank, device
        self.total, self.seg_pad = total, seg_pad
        self.muon_total = world * seg_pad
        self.adam_numel = total - self.muon_total
        group = dist.group.WORLD
        self.grad_arena = symm.empty(total, dtype=torch.float32, device=device)
        self.grad_arena.zero_()
        self._hG = symm.rendezvous(self.grad_arena, group)
        self._flags = symm.empty(self.MAX_RANKS * 4, dtype=torch.int32, device=device)
        self._flags.zero_()
        self._hF = symm.rendezvous(self._flags, group)
        self._g_ptrs = _ptr_array(list(self._hG.buffer_ptrs))
        self._f_ptrs = _ptr_array(list(self._hF.buffer_ptrs))
        # squared gradient norms: slot r of every rank's array receives rank r's share
        self.norms = symm.empty(self.MAX_RANKS, dtype=torch.float64, device=device)
        self.norms.zero_()
        self._hN = symm.rendezvous(self.norms, group)
        self._n_ptrs = _ptr_array(list(self._hN.buffer_ptrs))
        self._norm_part = torch.zeros(512, dtype=torch.float64, device=device)
        self._norm_done = torch.zeros(1, dtype=torch.int32, device=device)
        self._U: Optional[torch.Tensor] = None
        self._u_ptrs = None
        self.epoch = 0
        # NVLS in-switch reduction (multimem.ld_reduce) is opt-in
        self.use_multimem = (os.environ.get("IMF_B200_MULTIMEM", "0") == "1"
                             and bool(getattr(self._hG, "multicast_ptr", 0)))
        torch.cuda.synchronize(device)
        dist.barrier()          # flags are zero everywhere before the first epoch

    def update_arena(self, dtype: torch.dtype) -> torch.Tensor:
        import torch.distributed._symmetric_memory as symm

        self._U = symm.empty(self.muon_total, dtype=dtype, device=self.device)
        self._U.zero_()
        self._hU = symm.rendezvous(self._U, dist.group.WORLD)
        self._u_ptrs = _ptr_array(list(self._hU.buffer_ptrs))
        return self._U

    def _next(self) -> int:
        self.epoch += 1
        return self.epoch

    def _status(self):
        return K._ptr(K.status_word(self.device))

    def reduce_grads(self) -> None:
        """Muon segment -> owner, AdamW slice -> every rank (mean); the reduce pass also
        publishes every rank's squared norm of its reduced slices (``grad_sq_norm``)."""
        mc = vp(int(self._hG.multicast_ptr)) if self.use_multimem else None
        K._check(_lib.imf_comm_reduce(self._g_ptrs, self._f_ptrs, mc, self.rank, self.world,
                                      self.seg_pad, self.muon_total, self.adam_numel,
                                      self._next(), self._status(), self._n_ptrs,
                                      K._ptr(self._norm_part), K._ptr(self._norm_done),
                                      K._stream()), "imf_comm_reduce")
        shard = self.adam_numel // self.world
        K._check(_lib.imf_comm_gather(self._g_ptrs, self._f_ptrs, self.rank, self.world,
                                      self.muon_total, shard, 4, self._next(), self._status(),
                                      K._stream()), "imf_comm_gather")
        K.LAUNCHES.count += 2

    def all_gather_updates(self) -> None:
        K._check(_lib.imf_comm_gather(self._u_ptrs, self._f_ptrs, self.rank, self.world, 0,
                                      self.seg_pad, self._U.element_size(), self._next(),
                                      self._status(), K._stream()), "imf_comm_gather")
        K.LAUNCHES.count += 1

    def grad_sq_norm(self) -> torch.Tensor:
        """Squared global gradient norm (fp64 scalar on the device); valid after
        ``reduce_grads`` (its gather launch starts with a barrier that orders the slots)."""
        return self.norms[:self.world].sum()

    def apply_muon_updates(self, P: torch.Tensor, E: Optional[torch.Tensor], segs_dev: torch.Tensor,
                           nseg: int, max_numel: int, ema_w: float, clip: torch.Tensor) -> None:
        """p <- p (1 - lr wd) - lr s Phi (+ EMA) for every Muon parameter, Phi read from the
        owner's update arena over peer memory (no separate all-gather)."""
        K._check(_lib.imf_comm_muon_apply(self._u_ptrs, self._f_ptrs, self.rank, self.world,
                                          self.seg_pad, K._ptr(P), K._ptr(E), K._ptr(segs_dev), nseg,
                                          max_numel, float(ema_w), K._ptr(clip),
                                          int(self._U.dtype == torch.bfloat16), self._next(),
                                          self._status(), K._stream()), "imf_comm_muon_apply")
        K.LAUNCHES.count += 1

    def barrier(self) -> None:
        K._check(_lib.imf_comm_barrier(self._g_ptrs, self._f_ptrs, self.rank, self.world,
                                       self._next(), self._status(), K._stream()),
                 "imf_comm_barrier")
