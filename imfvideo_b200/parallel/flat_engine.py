"""Flat-arena optimizer engine for Moonlight (1 or N ranks).

All parameters, gradients, EMA weights and optimizer moments live in a few
contiguous fp32 arenas; ``p.data`` / ``p.grad`` / ``state[p][...]`` are views,
so ``state_dict()`` and checkpoints keep the reference layout while a whole
optimizer phase is a handful of launches instead of ~10 per parameter
(reference ``moonlight.py:395-469``, ``train.py:290-298``, ``:353-371``,
``:582``).

Arena layout (element offsets):

    [ Muon matrices owned by rank 0 | rank 1 | ... | rank W-1 | AdamW params ]

Each Muon segment is padded to ``seg_pad`` elements; inside a segment the
matrices are sorted by shape so every shape is one contiguous (k, n, m) batch
for Newton-Schulz.  The AdamW slice is padded to a multiple of 256 * W.

Per step:
  * gradient mean: Muon segment r is reduced onto rank r only, AdamW shard r
    likewise.  With peer memory this happens bucket by bucket (one bucket per
    transformer block) on a side stream while backward is still running, peers'
    contributions travel as bf16 and are summed in fp32; AdamW then runs on the
    shard and the updated parameters are gathered.  Without peer memory: NCCL /
    gloo on the same contiguous slices, AdamW replicated;
  * global norm -> device-side clip factor and skip flag (no host sync);
  * owner: momentum + batched Newton-Schulz on its segment; update all-gather;
    every rank applies ``p <- p (1 - lr wd) - lr s Phi`` (+ EMA) to all Muon
    parameters and AdamW (+ EMA) to the rest -> replicas stay bit-identical.

Deliberate difference from the reference optimizer (``moonlight.py`` ``_muon_step`` /
``_adamw_step`` skip parameters whose ``grad is None``): every parameter owns a
permanent, zero-filled gradient view in the arena, so a parameter that received no
gradient in a step is updated with a zero gradient (weight decay, moment decay).
All AdamW parameters share one step count (kept on the device, ``tcount``).
"""

from __future__ import annotations

import ctypes
import math
from collections import defaultdict
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..optim.moonlight import Moonlight, get_ns_coefficients, zeropower_via_newtonschulz5
from ..utils.versions import mark_written
from .grad_sync import GradSync
from .owner import assign_owners

SEG_DTYPE = np.dtype([("start", "<i8"), ("numel", "<i8"), ("a", "<f4"), ("b", "<f4")])


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class FlatEngine(GradSync):
    keeps_grad_views = True
    handles_ema = True

    def __init__(self, optimizer: Moonlight, net: torch.nn.Module, ema: Optional[torch.nn.Module],
                 rank: int, world: int, ema_decay: float = 0.0, mode: str = "fused_p2p",
                 ns_cuda_graph: bool = False, wire_dtype: str = "bfloat16",
                 overlap: bool = True):
        self.opt, self.net, self.ema = optimizer, net, ema
        self.wire_dtype, self.overlap = wire_dtype, bool(overlap)
        self.bucketed = False          # bucketed bf16 reduce + sharded AdamW (needs peer memory)
        self.armed = True              # False during all but the last micro-batch of a step
        self._launched: set = set()
        self._last_started: Optional[int] = None
        self.ns_cuda_graph = bool(ns_cuda_graph)
        self._ns_graph, self._ns_graph_launches, self._ns_eager_steps = None, 0, 0
        self.rank, self.world, self.mode = rank, world, mode
        self.ema_w = (1.0 - ema_decay) if ema is not None else 0.0
        name_of = {id(p): n for n, p in net.named_parameters()}
        ema_of = dict(ema.named_parameters()) if ema is not None else {}
        self.muon: List[Tuple[dict, torch.nn.Parameter]] = []
        self.adam: List[Tuple[dict, torch.nn.Parameter]] = []
        for g in optimizer.param_groups:
            for p in g["params"]:
                (self.muon if g["use_muon"] else self.adam).append((g, p))
        dev = next(net.parameters()).device
        self.device = dev
        self.cuda = dev.type == "cuda"
        shapes = [Moonlight._matrix_shape(p) for _, p in self.muon]
        self.shapes = shapes
        self.owner = assign_owners(shapes, world, optimizer.defaults["ns_steps"])
        # ---- layout ---------------------------------------------------------
        self.seg_items: List[List[int]] = [[] for _ in range(world)]
        for i, r in enumerate(self.owner):
            self.seg_items[r].append(i)
        for items in self.seg_items:                      # same-shape runs are contiguous
            items.sort(key=lambda i: (shapes[i], i))
        seg_numel = [sum(self.muon[i][1].numel() for i in it) for it in self.seg_items]
        self.seg_pad = _round_up(max(1, max(seg_numel)), 256)
        self.muon_off: Dict[int, int] = {}
        for r, items in enumerate(self.seg_items):
            off = r * self.seg_pad
            for i in items:
                self.muon_off[i] = off
                off += self.muon[i][1].numel()
        self.muon_total = world * self.seg_pad
        self.adam_off: List[int] = []
        off = self.muon_total
        for _, p in self.adam:
            self.adam_off.append(off)
            off += _round_up(p.numel(), 4)
        self.adam_numel = _round_up(off - self.muon_total, 256 * world)
        self.total = self.muon_total + self.adam_numel
        # ---- arenas ---------------------------------------------------------
        z = lambda n, dt=torch.float32: torch.zeros(n, dtype=dt, device=dev)
        self.comm = None
        if world > 1 and mode == "fused_p2p" and self.cuda:
            from ..ops import comm as comm_mod

            self.comm = comm_mod.try_create(world, rank, dev, self.total, self.seg_pad)
        self.bucketed = self.comm is not None and wire_dtype in ("bfloat16", "bf16")
        self.P = self.comm.make_param_arena() if self.bucketed else z(self.total)
        self.G = self.comm.grad_arena if self.comm is not None else z(self.total)
        self.E = z(self.total) if ema is not None else None
        self.M = z(self.muon_total)                       # momentum (own segment is live)
        self.A1, self.A2 = z(self.adam_numel), z(self.adam_numel)
        self.Dir = z(self.seg_pad)
        self.upd_dtype = (optimizer.defaults["ns_dtype"] or
                          (torch.bfloat16 if self.cuda else torch.float32))
        self.U = (self.comm.update_arena(self.upd_dtype) if self.comm is not None
                  else z(self.muon_total, self.upd_dtype))
        self.clip = z(2)                                  # [coef, skip flag]
        self.norm = z(1)
        # AdamW steps actually applied (skipped steps do not count); the kernels read the
        # bias corrections from here, the Python ints in ``state[p]["step"]`` follow it
        self.tcount = z(1)
        self._repoint(name_of, ema_of)
        self._muon_seg_host = np.zeros(len(self.muon), dtype=SEG_DTYPE)
        self._adam_seg_host = np.zeros(len(self.adam), dtype=SEG_DTYPE)
        for i, (_, p) in enumerate(self.muon):
            self._muon_seg_host[i]["start"] = self.muon_off[i]
            self._muon_seg_host[i]["numel"] = p.numel()
        for i, (_, p) in enumerate(self.adam):
            self._adam_seg_host[i]["start"] = self.adam_off[i]
            self._adam_seg_host[i]["numel"] = p.numel()
        self._muon_seg_dev = torch.zeros(max(1, len(self.muon)) * SEG_DTYPE.itemsize,
                                         dtype=torch.uint8, device=dev)
        self._adam_seg_dev = torch.zeros(max(1, len(self.adam)) * SEG_DTYPE.itemsize,
                                         dtype=torch.uint8, device=dev)
        self._max_muon = max([p.numel() for _, p in self.muon] + [1])
        self._max_adam = max([p.numel() for _, p in self.adam] + [1])
        self._lib = None
        if self.cuda:
            from ..ops import cuda as cu

            if cu.available():
                from ..ops import kernels as K

                if K._has("imf_adamw"):
                    self._lib = K._lib
                    self._K = K
                    self._bind()
        optimizer.distributed = self
        self.skipped_last = False
        self.buckets = self._build_buckets()
        if self.bucketed:
            self.comm.set_buckets(self.buckets)

    # -------------------------------------------------------------- buckets ---
    def _blocks(self):
        net = self.net
        return [b for name in ("shared_blocks", "u_heads", "v_heads")
                for b in getattr(net, name, [])]

    def _build_buckets(self):
        """One gradient bucket per transformer block (in forward order; backward finishes
        them in reverse) plus one for everything else.  A bucket is a list of arena ranges
        (start, numel, owner): a Muon matrix belongs to its owner rank, an AdamW range to
        the rank whose shard of the AdamW slice it falls in (ranges are cut at shard
        boundaries).  Every rank builds the same table."""
        blocks = self._blocks()
        bucket_of = {}
        for bi, blk in enumerate(blocks):
            for p in blk.parameters():
                bucket_of[id(p)] = bi
        nb = len(blocks) + 1
        buckets = [[] for _ in range(nb)]
        for i, (_, p) in enumerate(self.muon):
            buckets[bucket_of.get(id(p), nb - 1)].append(
                (self.muon_off[i], p.numel(), self.owner[i]))
        shard = self.adam_numel // self.world
        for i, (_, p) in enumerate(self.adam):
            lo, hi = self.adam_off[i], self.adam_off[i] + p.numel()
            while lo < hi:
                q = (lo - self.muon_total) // shard
                cut = min(hi, self.muon_total + (q + 1) * shard)
                buckets[bucket_of.get(id(p), nb - 1)].append((lo, cut - lo, int(q)))
                lo = cut
        if self.bucketed and self.overlap:
            from functools import partial

            for bi, blk in enumerate(blocks):
                if hasattr(blk, "fused_sinks"):
                    blk.fused_sinks().on_backward = partial(self._block_backward_started, bi)
        return buckets

    def _block_backward_started(self, bi: int) -> None:
        """Called by block ``bi``'s autograd node when its backward begins: the block whose
        backward ran before it has all its gradients in the arena by now (leaf accumulation
        runs before any other ready node), so its bucket goes out on the side stream while
        this block's backward computes."""
        if not (self.armed and self.bucketed):
            return
        prev, self._last_started = self._last_started, bi
        if prev is not None and prev != bi:
            self._launch_bucket(prev)

    def _launch_bucket(self, b: int) -> None:
        if b in self._launched:
            return
        if not self._launched:
            self.comm.begin_step()
        self._launched.add(b)
        self.comm.reduce_bucket(b)

    # ------------------------------------------------------------- set-up ---
    def _repoint(self, name_of, ema_of) -> None:
        opt = self.opt
        self._written = []        # every tensor a step writes through the arenas (see step())
        with torch.no_grad():
            def place(p, off):
                n = p.numel()
                self.P[off:off + n].copy_(p.detach().reshape(-1))
                p.data = self.P[off:off + n].view(p.shape)
                p.grad = self.G[off:off + n].view(p.shape)
                self._written.append(p)
                if self.E is not None:
                    q = ema_of.get(name_of[id(p)])
                    if q is not None:
                        self.E[off:off + n].copy_(q.detach().reshape(-1))
                        q.data = self.E[off:off + n].view(q.shape)
                        self._written.append(q)
            for i, (_, p) in enumerate(self.muon):
                place(p, self.muon_off[i])
                st = opt.state[p]
                o, n = self.muon_off[i], p.numel()
                if "momentum_buffer" in st:
                    self.M[o:o + n].copy_(st["momentum_buffer"].reshape(-1))
                st["momentum_buffer"] = self.M[o:o + n].view(self.shapes[i])
            for i, (_, p) in enumerate(self.adam):
                place(p, self.adam_off[i])
                st = opt.state[p]
                o, n = self.adam_off[i] - self.muon_total, p.numel()
                for key, arena in (("exp_avg", self.A1), ("exp_avg_sq", self.A2)):
                    if key in st:
                        arena[o:o + n].copy_(st[key].reshape(-1))
                    st[key] = arena[o:o + n].view(p.shape)
                st.setdefault("step", 0)

    def _bind(self) -> None:
        L = self._lib
        vp, ci, cl, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float
        L.imf_muon_momentum.restype = ci
        L.imf_muon_momentum.argtypes = [vp, vp, vp, cl, cf, ci, vp, vp]
        L.imf_muon_apply.restype = ci
        L.imf_muon_apply.argtypes = [vp, vp, ci, vp, vp, ci, cl, cl, cf, vp, vp]
        L.imf_adamw.restype = ci
        L.imf_adamw.argtypes = [vp, vp, vp, vp, vp, vp, ci, cl, cl, cf, cf, cf, cf, cf, vp, cf, vp,
                                cl, cl, vp]

    # ---------------------------------------------------------------- grads --
    def zero_grad(self) -> None:
        self.G.zero_()

    def _check_grad_views(self) -> None:
        """Autograd accumulates in place into existing ``.grad`` views; a grad
        that was set to None elsewhere is re-attached here."""
        for i, (_, p) in enumerate(self.muon):
            if p.grad is None or p.grad.data_ptr() != self.G.data_ptr() + self.muon_off[i] * 4:
                o, n = self.muon_off[i], p.numel()
                if p.grad is not None:
                    self.G[o:o + n].copy_(p.grad.reshape(-1))
                p.grad = self.G[o:o + n].view(p.shape)
        for i, (_, p) in enumerate(self.adam):
            if p.grad is None or p.grad.data_ptr() != self.G.data_ptr() + self.adam_off[i] * 4:
                o, n = self.adam_off[i], p.numel()
                if p.grad is not None:
                    self.G[o:o + n].copy_(p.grad.reshape(-1))
                p.grad = self.G[o:o + n].view(p.shape)

    @torch.no_grad()
    def sync(self) -> None:
        self._check_grad_views()
        w = self.world
        if w == 1:
            return
        if self.bucketed:
            # whatever the backward pass has not sent yet (at least the last block and the
            # non-block parameters), then this rank's share of the squared norm + barrier
            for b in range(len(self.buckets)):
                self._launch_bucket(b)
            self.comm.finish_norm()
            self._launched.clear()
            self._last_started = None
            return
        if self.comm is not None:
            self.comm.reduce_grads()            # own kernels: Muon segment -> owner, AdamW -> all
            return
        gm = self.G[:self.muon_total]
        ga = self.G[self.muon_total:]
        if dist.get_backend() == "nccl":
            own = gm[self.rank * self.seg_pad:(self.rank + 1) * self.seg_pad]
            dist.reduce_scatter_tensor(own, gm, op=dist.ReduceOp.SUM)
            own.div_(w)
        else:
            dist.all_reduce(gm, op=dist.ReduceOp.SUM)
            gm.div_(w)
        dist.all_reduce(ga, op=dist.ReduceOp.SUM)
        ga.div_(w)

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float) -> torch.Tensor:
        if self.world > 1 and self.comm is not None:
            sq = self.comm.grad_sq_norm()       # accumulated by the reduce kernel itself
        else:
            own = self.G[self.rank * self.seg_pad:(self.rank + 1) * self.seg_pad]
            sq = own.double().pow(2).sum()
            if self.world > 1:
                sq = sq.reshape(1)
                dist.all_reduce(sq, op=dist.ReduceOp.SUM)
                sq = sq[0]
            sq = sq + self.G[self.muon_total:].double().pow(2).sum()
        norm = sq.sqrt().float()
        finite = torch.isfinite(norm)
        coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        self.clip[0] = torch.where(finite, coef, torch.zeros_like(coef))
        self.clip[1] = (~finite).float()
        self.norm[0] = norm
        return norm

    # ----------------------------------------------------------------- step --
    def _refresh_groups(self) -> None:
        """Re-read which param-group dict each parameter belongs to.
        ``Optimizer.load_state_dict`` replaces ``param_groups`` with new dicts, and the
        trainer writes the scheduled learning rate into the current ones, so group
        references taken at construction go stale after a resume.  The parameter
        order (and with it every arena offset) never changes."""
        group_of = {id(p): g for g in self.opt.param_groups for p in g["params"]}
        self.muon = [(group_of[id(p)], p) for _, p in self.muon]
        self.adam = [(group_of[id(p)], p) for _, p in self.adam]

    def _upload_segments(self) -> None:
        wd_of = lambda g: g["weight_decay"]
        for i, (g, p) in enumerate(self.muon):
            lr = g["lr"]
            self._muon_seg_host[i]["a"] = 1.0 - lr * wd_of(g)
            self._muon_seg_host[i]["b"] = lr * Moonlight.muon_lr_scale(self.shapes[i],
                                                                       g["lr_scale_constant"])
        for i, (g, p) in enumerate(self.adam):
            self._adam_seg_host[i]["a"] = g["lr"]
            self._adam_seg_host[i]["b"] = 1.0 - g["lr"] * wd_of(g)
        for host, devbuf in ((self._muon_seg_host, self._muon_seg_dev),
                             (self._adam_seg_host, self._adam_seg_dev)):
            if len(host):
                devbuf[:host.nbytes].copy_(torch.from_numpy(host.view(np.uint8).reshape(-1)),
                                           non_blocking=True)

    @torch.no_grad()
    def step(self, opt: Moonlight) -> None:
        self._refresh_groups()
        use_k = self._lib is not None
        if use_k:
            self._upload_segments()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream) if use_k else None
        skip = self.clip[1]
        r = self.rank
        if self.muon:
            g0 = next(g for g, _ in self.muon)
            mu, nest = g0["momentum"], g0["nesterov"]
            own_g = self.G[r * self.seg_pad:(r + 1) * self.seg_pad]
            own_m = self.M[r * self.seg_pad:(r + 1) * self.seg_pad]
            if use_k:
                self._K._check(self._lib.imf_muon_momentum(
                    own_g.data_ptr(), own_m.data_ptr(), self.Dir.data_ptr(), self.seg_pad,
                    float(mu), int(nest), self.clip.data_ptr(), stream), "imf_muon_momentum")
                self._K.LAUNCHES.count += 1
            else:
                gc = own_g * self.clip[0]
                new_m = own_m * mu + gc
                own_m.copy_(torch.where(skip.bool(), own_m, new_m))
                self.Dir.copy_(gc + mu * own_m if nest else own_m)
            self._newton_schulz_phase(opt, g0, use_k)
            own_u = self.U[r * self.seg_pad:(r + 1) * self.seg_pad]
            fused_gather = self.world > 1 and self.comm is not None and use_k
            if self.world > 1 and not fused_gather:
                if self.comm is not None:
                    self.comm.all_gather_updates()
                elif dist.get_backend() == "nccl":
                    dist.all_gather_into_tensor(self.U, own_u)
                else:
                    parts = [torch.empty_like(own_u) for _ in range(self.world)]
                    dist.all_gather(parts, own_u.clone())
                    for q, part in enumerate(parts):
                        self.U[q * self.seg_pad:(q + 1) * self.seg_pad].copy_(part)
            if fused_gather:
                # the update all-gather happens inside the apply kernel (peer loads)
                self.comm.apply_muon_updates(self.P, self.E, self._muon_seg_dev, len(self.muon),
                                             self._max_muon, float(self.ema_w), self.clip)
            elif use_k:
                self._K._check(self._lib.imf_muon_apply(
                    self.P.data_ptr(), self.U.data_ptr(), int(self.upd_dtype == torch.bfloat16),
                    self.E.data_ptr() if self.E is not None else None,
                    self._muon_seg_dev.data_ptr(), len(self.muon), self._max_muon, 0,
                    float(self.ema_w), self.clip.data_ptr(), stream), "imf_muon_apply")
                self._K.LAUNCHES.count += 1
            else:
                keep = skip.bool()
                for i, (g, p) in enumerate(self.muon):
                    o, n = self.muon_off[i], p.numel()
                    lr = g["lr"]
                    sc = Moonlight.muon_lr_scale(self.shapes[i], g["lr_scale_constant"])
                    new = self.P[o:o + n] * (1 - lr * g["weight_decay"]) \
                        - lr * sc * self.U[o:o + n].float()
                    self.P[o:o + n].copy_(torch.where(keep, self.P[o:o + n], new))
        if self.adam:
            g0 = next(g for g, _ in self.adam)
            b1, b2 = g0["adamw_betas"]
            eps = g0["adamw_eps"]
            for _, p in self.adam:
                opt.state[p]["step"] += 1
            # the count on the device moves only when the step is applied (skip flag = 0),
            # so it stays exact even if the host never learns that a step was skipped
            self.tcount += 1.0 - skip
            if use_k:
                lo = hi = 0
                if self.bucketed:       # this rank's shard only; the others' arrive by gather
                    shard = self.adam_numel // self.world
                    lo = self.muon_total + r * shard
                    hi = lo + shard
                self._K._check(self._lib.imf_adamw(
                    self.P.data_ptr(), self.G.data_ptr(), self.A1.data_ptr(), self.A2.data_ptr(),
                    self.E.data_ptr() if self.E is not None else None,
                    self._adam_seg_dev.data_ptr(), len(self.adam), self._max_adam,
                    self.muon_total, float(b1), float(b2), float(eps), 1.0, 1.0,
                    self.clip.data_ptr(), float(self.ema_w), self.tcount.data_ptr(), lo, hi,
                    stream), "imf_adamw")
                self._K.LAUNCHES.count += 1
                if self.bucketed:
                    self.comm.gather_params(self.P, self.E, float(self.ema_w), self.clip)
            else:
                keep = skip.bool()
                t = self.tcount.double().clamp_min(1.0)
                bias1 = (1 - torch.tensor(b1, dtype=torch.float64) ** t).float()
                bias2 = (1 - torch.tensor(b2, dtype=torch.float64) ** t).float()
                sl = slice(self.muon_total, self.total)
                g = self.G[sl] * self.clip[0]
                m_new = self.A1 * b1 + (1 - b1) * g
                v_new = self.A2 * b2 + (1 - b2) * g * g
                den = (v_new / bias2).sqrt() + eps
                lr_vec = torch.zeros_like(g)
                dec_vec = torch.ones_like(g)
                for i, (gr, p) in enumerate(self.adam):
                    o, n = self.adam_off[i] - self.muon_total, p.numel()
                    lr_vec[o:o + n] = gr["lr"]
                    dec_vec[o:o + n] = 1 - gr["lr"] * gr["weight_decay"]
                new_p = self.P[sl] * dec_vec - lr_vec * (m_new / bias1) / den
                self.A1.copy_(torch.where(keep, self.A1, m_new))
                self.A2.copy_(torch.where(keep, self.A2, v_new))
                self.P[sl].copy_(torch.where(keep, self.P[sl], new_p))
        if not use_k and self.E is not None:
            lerp = self.E + self.ema_w * (self.P - self.E)
            self.E.copy_(torch.where(skip.bool(), self.E, lerp))
        # the arenas were written through raw pointers / other views: move the parameters'
        # version counters, which the blocks' cached bf16 weight copies are keyed on
        mark_written(self._written)

    def _newton_schulz_eager(self, opt: Moonlight, g0) -> None:
        """Batched Newton-Schulz per contiguous same-shape run of the owned segment:
        ``Dir`` (momentum direction) -> the owned slice of ``U``."""
        r = self.rank
        items = self.seg_items[r]
        j = 0
        own_u = self.U[r * self.seg_pad:(r + 1) * self.seg_pad]
        while j < len(items):
            shp = self.shapes[items[j]]
            k = j
            while k < len(items) and self.shapes[items[k]] == shp:
                k += 1
            lo = self.muon_off[items[j]] - r * self.seg_pad
            cnt = k - j
            n, m = shp
            batch = self.Dir[lo:lo + cnt * n * m].view(cnt, n, m)
            coeffs = get_ns_coefficients(n, m, steps=g0["ns_steps"], mode=g0["coeff_mode"],
                                         **opt._solve_kw)
            # the last iteration writes straight into the owned slice of the update arena
            zeropower_via_newtonschulz5(batch, steps=g0["ns_steps"], dtype=g0["ns_dtype"],
                                        coeffs=coeffs,
                                        out=own_u[lo:lo + cnt * n * m].view(cnt, n, m))
            j = k

    def _newton_schulz_phase(self, opt: Moonlight, g0, use_k: bool) -> None:
        """The phase is a fixed sequence of launches on fixed buffers (arena slices in, arena
        slices out, constant coefficients, no collective and no host read), so with
        ``ns_cuda_graph`` it is captured once, after one eager step has warmed every cache,
        and replayed as one graph launch afterwards."""
        if not (self.ns_cuda_graph and use_k and self.P.is_cuda):
            return self._newton_schulz_eager(opt, g0)
        if self._ns_graph is not None:
            self._ns_graph.replay()
            self._K.LAUNCHES.count += self._ns_graph_launches
            return
        if self._ns_eager_steps < 1:
            self._ns_eager_steps += 1
            return self._newton_schulz_eager(opt, g0)
        graph = torch.cuda.CUDAGraph()
        n0 = self._K.LAUNCHES.count
        try:
            # thread-local error mode: a pinned-memory allocation by a loader thread during
            # the capture must not invalidate it
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self._newton_schulz_eager(opt, g0)
        except RuntimeError:
            # nothing captured has run: do this step eagerly and stay eager from now on
            self._K.LAUNCHES.count = n0
            self.ns_cuda_graph = False
            return self._newton_schulz_eager(opt, g0)
        self._ns_graph_launches = self._K.LAUNCHES.count - n0
        self._K.LAUNCHES.count = n0
        self._ns_graph = graph
        self._ns_graph.replay()
        self._K.LAUNCHES.count += self._ns_graph_launches

    def undo_step_count(self) -> None:
        """Called by the trainer when it learns (from the device skip flag) that the last
        step was skipped: brings the Python ``step`` ints back in line with the device
        count, which is the one the update itself uses."""
        for _, p in self.adam:
            self.opt.state[p]["step"] -= 1

    def sync_step_count(self) -> None:
        """Host read of the device count into ``state[p]["step"]`` (before a checkpoint)."""
        if self.adam:
            t = int(round(float(self.tcount.item())))
            for _, p in self.adam:
                self.opt.state[p]["step"] = t

    # ---------------------------------------------------------- checkpoints --
    @torch.no_grad()
    def gather_state(self) -> None:
        self.sync_step_count()
        if self.world == 1 or not self.muon:
            return
        own = self.M[self.rank * self.seg_pad:(self.rank + 1) * self.seg_pad].clone()
        parts = [torch.empty_like(own) for _ in range(self.world)]
        dist.all_gather(parts, own)
        for q, part in enumerate(parts):
            self.M[q * self.seg_pad:(q + 1) * self.seg_pad].copy_(part)
        if self.bucketed:               # AdamW moments live on the shard owners
            shard = self.adam_numel // self.world
            for arena in (self.A1, self.A2):
                own = arena[self.rank * shard:(self.rank + 1) * shard].clone()
                parts = [torch.empty_like(own) for _ in range(self.world)]
                dist.all_gather(parts, own)
                for q, part in enumerate(parts):
                    arena[q * shard:(q + 1) * shard].copy_(part)

    @torch.no_grad()
    def after_load(self) -> None:
        """``load_state_dict`` replaced parameter / state tensors: pull the loaded
        values back into the arenas and re-attach the views."""
        name_of = {id(p): n for n, p in self.net.named_parameters()}
        ema_of = dict(self.ema.named_parameters()) if self.ema is not None else {}
        self._repoint(name_of, ema_of)
        self._refresh_groups()
        if self.adam:
            self.tcount.fill_(float(self.opt.state[self.adam[0][1]].get("step", 0)))

    def owner_table(self) -> List[int]:
        return list(self.owner)


def attach_engine(trainer, mode: str) -> FlatEngine:
    par = trainer.cfg.parallel
    if trainer.world > 1 and trainer.device.type == "cuda":
        try:
            from ..ops.comm_impl import set_peer_wait

            set_peer_wait(float(par.peer_wait_s))
        except Exception:
            pass
    return FlatEngine(trainer.optimizer, trainer.net, trainer.ema, trainer.rank, trainer.world,
                      trainer.cfg.run.ema_decay, mode,
                      ns_cuda_graph=getattr(trainer.cfg.optim, "ns_cuda_graph", False),
                      wire_dtype=par.wire_dtype, overlap=par.overlap_backward)
