"""Distributed Moonlight: gradient reduction, clipping and the optimizer step
with whole-matrix ownership.

Per step (every rank):
  1. Muon gradients are reduce-scattered so that each matrix's mean gradient
     lands ONLY at its owner (``parallel/owner.py``); AdamW gradients (a few
     percent of the parameters) are all-reduced.
  2. The global gradient norm is assembled from the owned pieces (one scalar
     all-reduce) and the clip factor is applied to the owned pieces.
  3. Each owner runs momentum + batched Newton-Schulz on its matrices only;
     the orthogonalised updates are all-gathered and every rank applies the
     same ``p <- p (1 - lr wd) - lr s Phi`` so replicas stay bit-identical.
  4. AdamW runs replicated.

The reference all-reduces one flat fp32 buffer after backward and repeats the
entire optimizer on every rank (reference ``train.py:353-371``,
``moonlight.py:395-437``).  On CUDA with peer access the two collectives of
step 1/3 are served by this repository's own reduce-scatter / all-gather
kernels over NVLink peer memory (``ops/comm.py``); on CPU (gloo) and as a
fallback the same layout goes through ``torch.distributed``.
"""

from __future__ import annotations

from collections import defaultdict
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..optim.moonlight import Moonlight
from .grad_sync import GradSync
from .owner import assign_owners


class DistributedMoonlight(GradSync):
    def __init__(self, optimizer: Moonlight, rank: int, world: int, mode: str = "fused_p2p",
                 wire_dtype: torch.dtype = torch.float32):
        self.opt, self.rank, self.world, self.mode = optimizer, rank, world, mode
        self.wire_dtype = wire_dtype
        self.muon: List[Tuple[dict, torch.nn.Parameter]] = []
        self.adam: List[torch.nn.Parameter] = []
        for g in optimizer.param_groups:
            for p in g["params"]:
                if g["use_muon"]:
                    self.muon.append((g, p))
                else:
                    self.adam.append(p)
        shapes = [Moonlight._matrix_shape(p) for _, p in self.muon]
        steps = optimizer.defaults["ns_steps"]
        self.owner = assign_owners(shapes, world, steps)
        self.shapes = shapes
        # owner-major layout: segment r = concatenation of rank r's matrices
        self.seg_items: List[List[int]] = [[] for _ in range(world)]
        for i, r in enumerate(self.owner):
            self.seg_items[r].append(i)
        self.seg_numel = [sum(self.muon[i][1].numel() for i in items) for items in self.seg_items]
        self.seg_pad = max(1, max(self.seg_numel))
        self.seg_pad = (self.seg_pad + 63) // 64 * 64
        self.offsets: Dict[int, int] = {}
        for items in self.seg_items:
            off = 0
            for i in items:
                self.offsets[i] = off
                off += self.muon[i][1].numel()
        dev = self.muon[0][1].device if self.muon else self.adam[0].device
        self.device = dev
        self.owned_grad: Optional[torch.Tensor] = None      # [seg_pad] fp32 mean gradient
        self.comm = None
        if mode == "fused_p2p" and dev.type == "cuda":
            from ..ops import comm as comm_mod

            self.comm = comm_mod.try_create(world, rank, dev, self.seg_pad)
        optimizer.distributed = self
        self._clip_coef: Optional[torch.Tensor] = None

    # ------------------------------------------------------------ helpers --
    def _pack_muon_grads(self) -> torch.Tensor:
        buf = torch.zeros(self.world, self.seg_pad, dtype=torch.float32, device=self.device)
        for r, items in enumerate(self.seg_items):
            for i in items:
                p = self.muon[i][1]
                if p.grad is not None:
                    o = self.offsets[i]
                    buf[r, o:o + p.numel()].copy_(p.grad.reshape(-1))
        return buf

    def _owned_view(self, i: int) -> torch.Tensor:
        o = self.offsets[i]
        p = self.muon[i][1]
        return self.owned_grad[o:o + p.numel()].view(self.shapes[i])

    # ---------------------------------------------------------------- sync --
    @torch.no_grad()
    def sync(self) -> None:
        w = self.world
        if self.muon:
            send = self._pack_muon_grads()
            if self.comm is not None:
                self.owned_grad = self.comm.reduce_scatter_mean(send)
            elif dist.get_backend() == "nccl":
                out = torch.empty(self.seg_pad, dtype=torch.float32, device=self.device)
                dist.reduce_scatter_tensor(out, send.view(-1), op=dist.ReduceOp.SUM)
                self.owned_grad = out.div_(w)
            else:        # gloo has no reduce-scatter: all-reduce and keep the owned row
                dist.all_reduce(send, op=dist.ReduceOp.SUM)
                self.owned_grad = send[self.rank].div(w)
        grads = [p.grad for p in self.adam if p.grad is not None]
        if grads:
            flat = torch.cat([g.reshape(-1).float() for g in grads])
            dist.all_reduce(flat, op=dist.ReduceOp.SUM)
            flat.div_(w)
            off = 0
            for g in grads:
                n = g.numel()
                g.copy_(flat[off:off + n].view_as(g))
                off += n

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float) -> torch.Tensor:
        """Global L2 norm over Muon (owned pieces, summed over ranks) and AdamW
        gradients; scales both by min(1, max_norm / (norm + 1e-6))."""
        sq_m = (self.owned_grad.double().pow(2).sum() if self.owned_grad is not None
                else torch.zeros((), dtype=torch.float64, device=self.device))
        dist.all_reduce(sq_m, op=dist.ReduceOp.SUM)
        grads = [p.grad for p in self.adam if p.grad is not None]
        sq_a = sum((g.double().pow(2).sum() for g in grads),
                   torch.zeros((), dtype=torch.float64, device=self.device))
        norm = (sq_m + sq_a).sqrt().float()
        coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        if self.owned_grad is not None:
            self.owned_grad.mul_(coef)
        if grads:
            torch._foreach_mul_(grads, coef)
        return norm

    # ---------------------------------------------------------------- step --
    @torch.no_grad()
    def step(self, opt: Moonlight) -> None:
        if self.muon:
            mine = self.seg_items[self.rank]
            by_group: Dict[int, List[int]] = defaultdict(list)
            for i in mine:
                by_group[id(self.muon[i][0])].append(i)
            upd_dtype = (torch.bfloat16 if self.device.type == "cuda"
                         and opt.defaults["ns_dtype"] is None else
                         (opt.defaults["ns_dtype"] or torch.float32))
            send = torch.zeros(self.seg_pad, dtype=upd_dtype, device=self.device)
            for items in by_group.values():
                group = self.muon[items[0]][0]
                dirs = []
                for i in items:
                    p = self.muon[i][1]
                    g = self._owned_view(i)
                    st = opt.state[p]
                    if "momentum_buffer" not in st:
                        st["momentum_buffer"] = torch.zeros_like(g)
                    buf = st["momentum_buffer"]
                    buf.mul_(group["momentum"]).add_(g)
                    dirs.append(g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf)
                for i, u in zip(items, opt._orthogonalize(group, dirs)):
                    o = self.offsets[i]
                    send[o:o + u.numel()].copy_(u.reshape(-1))
            if self.comm is not None:
                allu = self.comm.all_gather(send)
            else:
                allu = torch.empty(self.world, self.seg_pad, dtype=upd_dtype, device=self.device)
                dist.all_gather_into_tensor(allu.view(-1), send) if dist.get_backend() == "nccl" \
                    else dist.all_gather(list(allu.unbind(0)), send)
            for i, (group, p) in enumerate(self.muon):
                o = self.offsets[i]
                u = allu[self.owner[i], o:o + p.numel()].view(self.shapes[i])
                opt._muon_apply(group, p, u)
        for group in opt.param_groups:
            if not group["use_muon"]:
                opt._adamw_step(group)

    # --------------------------------------------------------- checkpoints --
    @torch.no_grad()
    def gather_state(self) -> None:
        """Give every rank every momentum buffer (collective) so rank 0 can
        write a complete, reference-compatible optimizer state."""
        if not self.muon:
            return
        send = torch.zeros(self.seg_pad, dtype=torch.float32, device=self.device)
        for i in self.seg_items[self.rank]:
            st = self.opt.state.get(self.muon[i][1], {})
            if "momentum_buffer" in st:
                o = self.offsets[i]
                send[o:o + st["momentum_buffer"].numel()].copy_(st["momentum_buffer"].reshape(-1))
        allb = [torch.empty_like(send) for _ in range(self.world)]
        dist.all_gather(allb, send)
        for i, (_g, p) in enumerate(self.muon):
            o = self.offsets[i]
            self.opt.state[p]["momentum_buffer"] = \
                allb[self.owner[i]][o:o + p.numel()].view(self.shapes[i]).clone()

    def after_load(self) -> None:
        return

    def owner_table(self) -> List[int]:
        return list(self.owner)


def attach_distributed(trainer, mode: str) -> DistributedMoonlight:
    wire = getattr(torch, trainer.cfg.parallel.wire_dtype)
    return DistributedMoonlight(trainer.optimizer, trainer.rank, trainer.world, mode, wire)
