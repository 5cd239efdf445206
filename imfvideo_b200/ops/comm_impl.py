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
    _lib.imf_comm_bucket_pack.restype = ci
    _lib.imf_comm_bucket_pack.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp, vp]
    _lib.imf_comm_bucket_reduce.restype = ci
    _lib.imf_comm_bucket_reduce.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp, vp, vp]
    _lib.imf_comm_norm_finish.restype = ci
    _lib.imf_comm_norm_finish.argtypes = [vp, vp, vp, ci, ci, ci, ci, vp, vp]
    _lib.imf_comm_param_gather.restype = ci
    _lib.imf_comm_param_gather.argtypes = [vp, vp, vp, vp, ci, ci, cl, cl, ctypes.c_float, vp, ci,
                                           vp, vp]

    _lib.imf_comm_max.restype = ci
    _lib.imf_comm_max.argtypes = [vp, vp, vp, ci, ci, ci, ci, vp, vp]

MAX_BUCKETS = 64
BUCKET_BX = 8
FLAG_INTS = 4 * 16 + MAX_BUCKETS * 16
RANGE_DTYPE = [("start", "<i8"), ("numel", "<i8"), ("owner", "<i4"), ("pad", "<i4")]


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
        self._flags = symm.empty(FLAG_INTS, dtype=torch.int32, device=device)
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
        # bucketed bf16 path (set up by ``set_buckets``)
        self.wire: Optional[torch.Tensor] = None
        self.param_arena: Optional[torch.Tensor] = None
        self.bucket_step = 0
        self.side_stream = torch.cuda.Stream(device)
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

    # ------------------------------------------------------- bucketed bf16 path --
    def make_param_arena(self) -> torch.Tensor:
        """fp32 parameter arena in symmetric memory: after the sharded AdamW the other ranks
        read this rank's updated shard from it."""
        import torch.distributed._symmetric_memory as symm

        self.param_arena = symm.empty(self.total, dtype=torch.float32, device=self.device)
        self.param_arena.zero_()
        self._hP = symm.rendezvous(self.param_arena, dist.group.WORLD)
        self._p_ptrs = _ptr_array(list(self._hP.buffer_ptrs))
        return self.param_arena

    def set_buckets(self, buckets) -> None:
        """``buckets``: list (one entry per bucket, same on every rank) of lists of
        (start, numel, owner) arena ranges.  Allocates the bf16 wire arena."""
        import numpy as np
        import torch.distributed._symmetric_memory as symm

        if len(buckets) > MAX_BUCKETS:
            raise RuntimeError(f"at most {MAX_BUCKETS} gradient buckets")
        self.wire = symm.empty(self.total, dtype=torch.bfloat16, device=self.device)
        self.wire.zero_()
        self._hW = symm.rendezvous(self.wire, dist.group.WORLD)
        self._w_ptrs = _ptr_array(list(self._hW.buffer_ptrs))
        rows, self._bk = [], []
        for b in buckets:
            self._bk.append((len(rows), len(b)))
            rows += [(int(s), int(n), int(o), 0) for s, n, o in b]
        host = np.array(rows, dtype=np.dtype(RANGE_DTYPE)) if rows else \
            np.zeros(0, dtype=np.dtype(RANGE_DTYPE))
        self._ranges = torch.from_numpy(host.view(np.uint8).reshape(-1).copy()).to(self.device)
        self._range_bytes = np.dtype(RANGE_DTYPE).itemsize
        self._parts = torch.zeros(max(1, len(rows)) * BUCKET_BX, dtype=torch.float64,
                                  device=self.device)
        self._pack_done = torch.zeros(MAX_BUCKETS, dtype=torch.int32, device=self.device)
        self._n_parts = len(rows) * BUCKET_BX
        torch.cuda.synchronize(self.device)
        dist.barrier()

    def begin_step(self) -> None:
        self.bucket_step += 1

    def reduce_bucket(self, b: int, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Pack + reduce bucket ``b`` of the current step on ``stream`` (default: the side
        stream, ordered after everything queued so far on the current stream)."""
        first, n = self._bk[b]
        if n == 0:
            return
        st = stream or self.side_stream
        if st != torch.cuda.current_stream(self.device):
            st.wait_stream(torch.cuda.current_stream(self.device))
        sp = vp(st.cuda_stream)
        rng = vp(self._ranges.data_ptr() + first * self._range_bytes)
        K._check(_lib.imf_comm_bucket_pack(self._f_ptrs, K._ptr(self.grad_arena), K._ptr(self.wire),
                                           rng, n, self.rank, self.world, b, self.bucket_step,
                                           vp(self._pack_done.data_ptr() + 4 * b), sp),
                 "imf_comm_bucket_pack")
        K._check(_lib.imf_comm_bucket_reduce(self._f_ptrs, self._w_ptrs, K._ptr(self.grad_arena),
                                             rng, n, self.rank, self.world, b, self.bucket_step,
                                             self._status(),
                                             vp(self._parts.data_ptr() + 8 * first * BUCKET_BX),
                                             sp), "imf_comm_bucket_reduce")
        K.LAUNCHES.count += 2

    def finish_norm(self) -> None:
        """Join the side stream, publish this rank's squared-norm share, barrier."""
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self.side_stream)
        K._check(_lib.imf_comm_norm_finish(self._f_ptrs, self._n_ptrs, K._ptr(self._parts),
                                           self._n_parts, self.rank, self.world, self._next(),
                                           self._status(), K._stream()), "imf_comm_norm_finish")
        K.LAUNCHES.count += 1

    def gather_params(self, P: torch.Tensor, E: Optional[torch.Tensor], ema_w: float,
                      clip: torch.Tensor) -> None:
        """Every rank's updated AdamW shard -> every rank's parameter arena (+ EMA)."""
        assert P.data_ptr() == self.param_arena.data_ptr()
        shard = self.adam_numel // self.world
        K._check(_lib.imf_comm_param_gather(self._f_ptrs, self._p_ptrs, K._ptr(P), K._ptr(E),
                                            self.rank, self.world, self.muon_total, shard,
                                            float(ema_w), K._ptr(clip), self._next(),
                                            self._status(), K._stream()), "imf_comm_param_gather")
        K.LAUNCHES.count += 1

    MAX_STATS = 4096

    def max_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Element-wise maximum over ranks of a small fp32 tensor, by this library's kernel
        over peer memory (no NCCL, no host read).  Returns a new tensor of x's shape."""
        n = x.numel()
        if n > self.MAX_STATS:
            raise ValueError(f"max_reduce holds at most {self.MAX_STATS} values")
        if getattr(self, "_stat_in", None) is None:
            import torch.distributed._symmetric_memory as symm

            self._stat_in = symm.empty(self.MAX_STATS, dtype=torch.float32, device=self.device)
            self._stat_in.zero_()
            self._hS = symm.rendezvous(self._stat_in, dist.group.WORLD)
            self._s_ptrs = _ptr_array(list(self._hS.buffer_ptrs))
        self._stat_in[:n].copy_(x.reshape(-1).float())
        out = torch.empty(n, dtype=torch.float32, device=self.device)
        K._check(_lib.imf_comm_max(self._s_ptrs, self._f_ptrs, K._ptr(out), n, self.rank,
                                   self.world, self._next(), self._status(), K._stream()),
                 "imf_comm_max")
        K.LAUNCHES.count += 1
        return out.view(x.shape)

    def barrier(self) -> None:
        K._check(_lib.imf_comm_barrier(self._g_ptrs, self._f_ptrs, self.rank, self.world,
                                       self._next(), self._status(), K._stream()),
                 "imf_comm_barrier")
