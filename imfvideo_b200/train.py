"""iMF video training runtime: ``Trainer`` (one object = one rank) and ``main``.

Launch: ``python -m imfvideo_b200.train [group.key=value ...]`` or
``torchrun --nproc-per-node N -m imfvideo_b200.train ...``.

Step anatomy follows the reference loop (``train.py:539-616``): grad-accum
micro-steps, gradient averaging over ranks, per-group lr with muP width
multipliers, global-norm clip, non-finite-step skip, optimizer step, QK-clip,
EMA, logging, checkpoint.  Replicas start from rank 0's weights (the
reference seeds each rank differently and never broadcasts,
``train.py:391-396``); the per-rank seed only drives data noise.
"""

from __future__ import annotations

import copy
import math
import os
import sys
import time
from functools import partial
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import config as config_mod
from .config import Config, config_as_dict
from .data.dataset import DevicePrefetcher, InfiniteLoader, build_loader
from .loss import IMFVideoLoss
from .models import imf_dit_video as M
from .optim.moonlight import build_moonlight
from .parallel import dist as pdist
from .parallel.grad_sync import FlatAllReduce, GradSync, NoSync
from .utils import checkpoint as ckpt_mod
from .utils.ema import ema_update
from .utils.schedule import lr_at as _lr_at
from .utils.timers import PhaseTimer
from .utils.versions import mark_written

D0 = 256.0   # width the learning rates were tuned at (muP reference width)


# ------------------------------------------------------------- builders ---
def build_attn_impl(cfg: Config):
    """Map ``model.attn_impl`` to an attention plug-in (function on duals, or
    a module factory for the SLA2 family); reference ``train.py:103-165``."""
    m = cfg.model
    name = m.attn_impl
    if name == "flash_jvp":
        return M.flash_jvp_attention
    if name == "sdpa_flash":
        return M.sdpa_flash_attention
    if name == "sdpa":
        return M.sdpa_math_attention
    if name == "sla2_jvp":
        from .models.sla2 import SLA2AttentionImpl

        return partial(SLA2AttentionImpl, topk=m.sla2_topk, bq=m.sla2_bq, bk=m.sla2_bk,
                       alpha_init=m.sla2_alpha_init)
    if name == "sla2_cube_qat":
        from .models.sla2 import SLA2CubeQATAttentionImpl

        pt, ph, pw = m.patch_size
        lh, lw = cfg.data.latent_size
        return partial(SLA2CubeQATAttentionImpl,
                       grid=(cfg.data.latent_frames // pt, lh // ph, lw // pw),
                       tile=tuple(m.sla2_tile), topk=m.sla2_topk, alpha_init=m.sla2_alpha_init)
    raise ValueError(f"unknown attn_impl {name!r}")


def build_model(cfg: Optional[Config] = None) -> Tuple[M.IMFDiTVideo, int, str]:
    cfg = cfg or config_mod.config
    m = cfg.model
    attn = build_attn_impl(cfg)
    net = M.IMFDiTVideo(
        input_size=tuple(cfg.data.latent_size) if not isinstance(cfg.data.latent_size, int)
        else cfg.data.latent_size,
        num_frames=cfg.data.latent_frames, patch_size=tuple(m.patch_size),
        in_channels=m.in_channels, hidden_size=m.hidden_size, depth=m.depth,
        num_heads=m.num_heads, num_classes=m.num_classes, aux_head_depth=m.aux_head_depth,
        q_lora_rank=m.q_lora_rank, kv_lora_rank=m.kv_lora_rank,
        qk_nope_head_dim=m.qk_nope_head_dim, qk_rope_head_dim=m.qk_rope_head_dim,
        v_head_dim=m.v_head_dim, mlp_ratio=m.mlp_ratio, num_class_tokens=m.num_class_tokens,
        num_time_tokens=m.num_time_tokens, num_cfg_tokens=m.num_cfg_tokens,
        num_interval_tokens=m.num_interval_tokens, freq_embedding_size=m.freq_embedding_size,
        token_init_constant=m.token_init_constant,
        embedding_init_constant=m.embedding_init_constant,
        weight_init_constant=m.weight_init_constant, rmsnorm_eps=m.rmsnorm_eps,
        rope_theta=m.rope_theta, eval_mode=m.eval_mode, attn_impl=attn,
        attn_res_block_size=m.attn_res_block_size, situ_beta=m.situ_beta,
        situ_linear_beta=m.situ_linear_beta, mla_use_output_gate=m.mla_use_output_gate,
        grad_checkpoint=m.grad_checkpoint)
    n = sum(p.numel() for p in net.parameters())
    assert n <= m.max_params, f"model has {n / 1e6:.1f}M params, cap {m.max_params / 1e6:.0f}M"
    return net, n, getattr(attn, "__name__", str(attn))


def build_optimizer(net, o, device, verbose=False):
    if o.optimizer == "moonlight":
        if verbose and o.weight_decay < 1e-3:
            print(f"WARNING: moonlight with weight_decay={o.weight_decay:g}; the Muon "
                  "branch is effectively undecayed", flush=True)
        return build_moonlight(
            net, lr=o.lr, weight_decay=o.weight_decay, momentum=o.muon_momentum,
            nesterov=o.muon_nesterov, ns_steps=o.muon_ns_steps,
            lr_scale_constant=o.muon_lr_scale_constant, adamw_betas=tuple(o.betas),
            coeff_mode=o.muon_coeff_mode, coeff_samples=o.muon_coeff_samples,
            coeff_iters=o.muon_coeff_iters, coeff_lr=o.muon_coeff_lr,
            coeff_seed=o.muon_coeff_seed, verbose=verbose)
    if o.optimizer == "adamw":
        return torch.optim.AdamW(net.parameters(), lr=o.lr, weight_decay=o.weight_decay,
                                 betas=tuple(o.betas),
                                 fused=o.fused_adamw and device.type == "cuda")
    raise ValueError(f"unknown optimizer {o.optimizer!r}")


def apply_lr_width_groups(optimizer, net, hidden_size: int, verbose=False) -> None:
    """Split the optimizer's groups by parameter NAME into muP width classes
    and store the factor as ``group["lr_width_mult"]`` (reference
    ``train.py:444-478``): Muon score heads (``_res_proj``) and AdamW output
    projections d0/d; other Muon matrices sqrt(d0/d); everything else 1."""
    ratio = hidden_size / D0
    name_of = {id(p): n for n, p in net.named_parameters()}
    groups = []
    for g in optimizer.param_groups:
        buckets: Dict[float, List] = {}
        for p in g["params"]:
            nm = name_of.get(id(p), "")
            if g.get("use_muon") and "_res_proj" in nm:
                mult = 1.0 / ratio
            elif g.get("use_muon"):
                mult = ratio ** -0.5
            elif "final_layer" in nm and ".norm." not in nm:
                mult = 1.0 / ratio
            else:
                mult = 1.0
            buckets.setdefault(mult, []).append(p)
        for mult, ps in buckets.items():
            ng = {k: v for k, v in g.items() if k != "params"}
            ng["params"], ng["lr_width_mult"] = ps, mult
            groups.append(ng)
    optimizer.param_groups = groups
    if verbose:
        for g in groups:
            print(f"lr group: muon={g.get('use_muon', False)} mult={g['lr_width_mult']:.3f} "
                  f"params={sum(p.numel() for p in g['params']) / 1e6:.2f}M", flush=True)


def lr_at(step: int, cfg: Optional[Config] = None) -> float:
    return _lr_at(step, (cfg or config_mod.config).optim)


@torch.no_grad()
def qk_clip(net, tau: float, world: int = 1, skip: Optional[torch.Tensor] = None,
            ema=None, ema_w: float = 0.0, as_tensors: bool = False, max_reduce=None):
    """MuonClip: heads whose max logit exceeded ``tau`` (nats) get the rope
    rows of ``q_b_proj`` scaled by tau / S_max.  All modules' per-head stats
    are reduced in ONE batched MAX all-reduce (the reference does an
    all-reduce and two host syncs per module, ``train.py:301-350``).

    ``skip``: the optimizer's device word [clip factor, skip flag]; when the
    flag is set (non-finite gradient norm) nothing is rescaled, as in the
    reference, which clips only inside its finite branch (``train.py:583-592``).
    A non-finite statistic clips nothing either.  ``ema`` / ``ema_w``: when the
    optimizer already folded the un-clipped weights into the EMA model (fused
    update kernels), the clipped rows of the EMA copy are corrected so the result
    equals the reference order step -> clip -> EMA.

    ``max_reduce``: callable doing the element-wise MAX over ranks (the peer-memory
    kernel of the optimizer engine); default ``torch.distributed.all_reduce``.

    Returns (#clipped heads, global max logit) as Python numbers, or as two
    device scalars with ``as_tensors`` (no host read)."""
    # the module walk, the EMA pairing and (below) the kernel's pointer table are the same
    # every step: they are built once per (net, ema) and kept on the net
    cache = net.__dict__.setdefault("_qk_clip_cache", {})
    key = (id(ema) if (ema is not None and ema_w > 0) else None)
    if cache.get("key", "unset") != key:
        cache.clear()
        cache["key"] = key
        named = [(n, m) for n, m in net.named_modules() if isinstance(m, M.MLAAttention)]
        ema_mods = dict(ema.named_modules()) if key is not None else {}
        cache["named"] = [(m, ema_mods.get(n)) for n, m in named]
    pairs = [(m, e) for m, e in cache["named"]
             if getattr(m.attn_impl, "logit_max_log2", None) is not None]
    if not pairs:
        if as_tensors:
            z = cache.get("zero")
            if z is None:
                z = cache["zero"] = torch.zeros((), device=next(net.parameters()).device)
            return z, z
        return 0, 0.0
    mods = [m for m, _ in pairs]
    emas = [e for _, e in pairs]
    rows = [m.attn_impl.logit_max_log2.float() for m in mods]
    buf = cache.get("stats")
    if buf is None or buf.shape != (len(rows),) + tuple(rows[0].shape) or buf.device != rows[0].device:
        buf = cache["stats"] = torch.empty(len(rows), *rows[0].shape, dtype=torch.float32,
                                           device=rows[0].device)
        cache.pop("table", None)
    stats = torch.stack(rows, out=buf)                                          # (n, H)
    if world > 1:
        if max_reduce is not None:
            stats = max_reduce(stats)
        else:
            dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    fused = _qk_clip_kernel(mods, emas, stats, tau, skip, ema_w,
                            cache if (world == 1 or max_reduce is None) else None)
    if fused is not None:
        n_hot, s_max = fused
    else:
        s_nat = stats * math.log(2.0)
        finite = torch.isfinite(s_nat)
        gamma = (tau / s_nat.clamp_min(1e-20)).clamp(max=1.0)
        gamma = torch.where(finite, gamma, torch.ones_like(gamma))
        if skip is not None:
            gamma = torch.where(skip[1].to(gamma.device) != 0, torch.ones_like(gamma), gamma)
        for m, e, g in zip(mods, emas, gamma):
            dn = m.qk_nope_head_dim
            w = m.q_b_proj.weight.view(m.num_heads, m.qk_head_dim, -1)
            gg = g.to(w.dtype).view(-1, 1, 1)
            if e is not None:
                ew = e.q_b_proj.weight.view(m.num_heads, m.qk_head_dim, -1)
                ew[:, dn:, :] += ema_w * (gg - 1.0) * w[:, dn:, :]
            w[:, dn:, :] *= gg
        n_hot = (gamma < 1.0).sum().float()
        s_max = torch.where(finite, s_nat, torch.zeros_like(s_nat)).max()
    if as_tensors:
        return n_hot, s_max
    n, mx = torch.stack([n_hot.float(), s_max.float()]).tolist()
    return int(n), float(mx)


def _qk_clip_kernel(mods, emas, stats: torch.Tensor, tau: float, skip, ema_w: float,
                    cache: Optional[dict] = None):
    """All modules in one launch of the library's kernel (fp32 contiguous weights on a GPU);
    None when that does not apply.  Returns two device scalars.  ``cache``: a dict in which the
    device copy of the pointer table is kept while ``stats`` and the weights stay where they
    are (the caller passes its persistent statistics buffer then)."""
    w0 = mods[0].q_b_proj.weight
    if not w0.is_cuda or any(m.q_b_proj.weight.dtype != torch.float32
                             or not m.q_b_proj.weight.is_contiguous() for m in mods):
        return None
    try:
        from .ops import cuda as cu
        if not cu.available():
            return None
        from .ops import kernels as K
    except Exception:
        return None
    if not K._has("imf_qk_clip"):
        return None
    import ctypes

    import numpy as np

    rec = np.dtype([("w", "<u8"), ("stat", "<u8"), ("H", "<i4"), ("hd", "<i4"), ("dn", "<i4"),
                    ("cols", "<i4"), ("ema", "<u8")])
    stats = stats.contiguous()
    sig = (stats.data_ptr(), tuple(m.q_b_proj.weight.data_ptr() for m in mods),
           tuple(0 if e is None else e.q_b_proj.weight.data_ptr() for e in emas))
    table = None
    if cache is not None and cache.get("table_sig") == sig:
        table = cache.get("table")
    if table is None:
        host = np.zeros(len(mods), dtype=rec)
        for i, (m, e) in enumerate(zip(mods, emas)):
            w = m.q_b_proj.weight
            ew = 0
            if e is not None and e.q_b_proj.weight.dtype == torch.float32 \
                    and e.q_b_proj.weight.is_contiguous():
                ew = e.q_b_proj.weight.data_ptr()
            host[i] = (w.data_ptr(), stats[i].data_ptr(), m.num_heads, m.qk_head_dim,
                       m.qk_nope_head_dim, w.shape[1], ew)
        table = torch.from_numpy(host.view(np.uint8).reshape(-1).copy()).to(w0.device)
        if cache is not None:
            cache["table"], cache["table_sig"] = table, sig
    summary = torch.zeros(2, dtype=torch.float32, device=w0.device)
    lib = K._lib
    lib.imf_qk_clip.restype = ctypes.c_int
    lib.imf_qk_clip.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                ctypes.c_void_p]
    K._check(lib.imf_qk_clip(K._ptr(table), len(mods), max(m.num_heads for m in mods), float(tau),
                             K._ptr(summary), K._ptr(skip), float(ema_w), K._stream()),
             "imf_qk_clip")
    K.LAUNCHES.count += 1
    # the kernel wrote the weights through raw pointers: move their version counters
    mark_written([m.q_b_proj.weight for m in mods] +
                 [e.q_b_proj.weight for e in emas if e is not None])
    return summary[0], summary[1]


# --------------------------------------------------------------- trainer ---
class Trainer:
    """Owns model, EMA, loss, optimizer, gradient sync and checkpoints for one
    rank.  ``train_step(latents, labels)`` is the public per-step call: it
    accepts host (pinned) or device tensors and returns a dict of Python
    floats (one device->host read per step)."""

    def __init__(self, cfg: Optional[Config] = None, rank: int = 0, world: int = 1,
                 device: Optional[torch.device] = None, verbose: Optional[bool] = None):
        self.cfg = cfg = cfg or config_mod.config
        self.rank, self.world = rank, world
        self.device = device or pdist.resolve_device()[0]
        self.verbose = (rank == 0) if verbose is None else verbose
        torch.manual_seed(cfg.run.seed)          # same init everywhere ...
        net, self.num_params, self.attn_name = build_model(cfg)
        self.net = net.to(self.device, dtype=getattr(torch, cfg.run.master_dtype))
        if cfg.loss.autocast_bf16 and self.device.type == "cuda":
            self.net.compute_dtype = torch.bfloat16
        if world > 1 and cfg.parallel.broadcast_init:
            pdist.broadcast_module(self.net, src=0)   # ... and enforced
        torch.manual_seed(cfg.run.seed + 1 + rank)     # data noise differs per rank
        self.ema = None
        if cfg.run.ema_decay > 0:
            self.ema = copy.deepcopy(self.net).eval().requires_grad_(False)
        lc = cfg.loss
        self.loss_mod = IMFVideoLoss(
            self.net, cfg.model.num_classes, P_mean=lc.P_mean, P_std=lc.P_std,
            data_proportion=lc.data_proportion, cfg_beta=lc.cfg_beta,
            class_dropout_prob=lc.class_dropout_prob, s_max=lc.cfg_s_max, norm_p=lc.norm_p,
            norm_eps=lc.norm_eps, loss_v_weight=lc.loss_v_weight,
            jvp_impl=lc.jvp_impl, stratified_time=lc.stratified_time,
            stratified_interval=lc.stratified_interval,
            strat_group=(cfg.data.batch_size_per_gpu * cfg.optim.grad_accum
                         if lc.strat_group_auto else 0),
            autocast_bf16=lc.autocast_bf16 and self.device.type == "cuda")
        o = cfg.optim
        assert o.grad_accum >= 1
        self.optimizer = build_optimizer(self.net, o, self.device, verbose=self.verbose)
        apply_lr_width_groups(self.optimizer, self.net, cfg.model.hidden_size, self.verbose)
        self.grad_sync: GradSync = self._build_grad_sync()
        self.step = 0
        self.timer = PhaseTimer(enabled=cfg.run.profile_phases)
        self._early_host = self._late_host = self._early_ev = self._late_ev = None
        self._late_pending = False
        if cfg.run.deterministic and self.device.type == "cuda":
            from .ops import kernels as _K
            _K.set_deterministic(True)
        self._nan_dumped = False
        self.last: Dict[str, Any] = {}
        if self.verbose:
            a = self.net.shared_blocks[0].attn if len(self.net.shared_blocks) else \
                self.net.u_heads[0].attn
            print(f"model: {self.num_params / 1e6:.1f}M params, world={world}, "
                  f"device={self.device}, attn={self.attn_name}", flush=True)
            print(f"MLA: heads={a.num_heads} q_lora={a.q_lora_rank} kv_lora={a.kv_lora_rank} "
                  f"qk_nope={a.qk_nope_head_dim} qk_rope={a.qk_rope_head_dim} "
                  f"v={a.v_head_dim}", flush=True)

    def _build_grad_sync(self) -> GradSync:
        mode = self.cfg.parallel.grad_sync
        if self.cfg.optim.optimizer == "moonlight" and mode != "nccl_flat":
            from .parallel.flat_engine import attach_engine

            return attach_engine(self, mode)      # flat arenas; owner-partitioned when world > 1
        if self.world == 1:
            return NoSync()
        return FlatAllReduce(list(self.net.parameters()), self.world)

    # ----------------------------------------------------------- stepping --
    def _to_device(self, latents, labels):
        labels = torch.as_tensor(labels)
        if latents.device != self.device:
            latents = latents.to(self.device, non_blocking=True)
        if labels.device != self.device:
            labels = labels.to(self.device, non_blocking=True)
        return latents.to(getattr(torch, self.cfg.run.master_dtype)), labels

    def micro_step(self, latents, labels) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        """Loss forward + backward of one micro-batch (gradients accumulate)."""
        latents, labels = self._to_device(latents, labels)
        with self.timer.phase("loss_fwd"):
            loss, parts = self.loss_mod(latents, labels)
        with self.timer.phase("backward"):
            (loss / self.cfg.optim.grad_accum).backward()
        parts["_latents"], parts["_labels"] = latents, labels
        return loss.detach(), parts

    @torch.no_grad()
    def _grad_norm_and_clip(self, max_norm: float) -> torch.Tensor:
        if hasattr(self.grad_sync, "clip_grad_norm_"):
            return self.grad_sync.clip_grad_norm_(max_norm)
        return torch.nn.utils.clip_grad_norm_(self.net.parameters(), max_norm)

    def optimizer_step(self, early=None) -> Dict[str, Any]:
        """Sync, lr, clip, (skip if non-finite) step, QK-clip, EMA.  With the
        flat engine the non-finite check happens on the device (skip flag), so
        nothing here waits for the GPU; statistics are returned as tensors.
        ``early(grad_norm, skipped)`` is called (flat engine only) once the norm and the skip
        flag are enqueued and before the update kernels are."""
        o = self.cfg.optim
        eng = self.grad_sync if getattr(self.grad_sync, "handles_ema", False) else None
        with self.timer.phase("grad_sync"):
            self.grad_sync.sync()
        lr = _lr_at(self.step, o)
        for g in self.optimizer.param_groups:
            g["lr"] = lr * g.get("lr_width_mult", 1.0)
        with self.timer.phase("optimizer"):
            grad_norm = self._grad_norm_and_clip(o.grad_clip)
            if eng is not None:
                if early is not None:
                    early(grad_norm, eng.clip[1])
                self.optimizer.step()
                skipped = eng.clip[1]
                # the fused update kernels have already folded the new weights into the
                # EMA; the clip corrects the EMA rows it rescales and honours the skip flag
                comm = getattr(eng, "comm", None)
                n_hot, s_max = qk_clip(self.net, o.qk_clip_tau, self.world, skip=eng.clip,
                                       ema=self.ema, ema_w=eng.ema_w, as_tensors=True,
                                       max_reduce=comm.max_reduce if comm is not None else None)
            else:
                finite = bool(torch.isfinite(grad_norm))
                skipped = torch.tensor(float(not finite))
                if finite:
                    self.optimizer.step()
                    n_hot, s_max = qk_clip(self.net, o.qk_clip_tau, self.world)
                    if self.ema is not None:
                        ema_update(self.ema, self.net, self.cfg.run.ema_decay)
                else:
                    n_hot, s_max = 0, float("nan")
                    self._report_bad_grads()
        if eng is not None:
            eng.zero_grad()
        else:
            self.optimizer.zero_grad(set_to_none=True)
        self.step += 1
        return {"lr": lr, "grad_norm": grad_norm, "skipped": skipped,
                "qk_hot": n_hot, "qk_smax": s_max}

    def _report_bad_grads(self) -> None:
        if not self.verbose:
            return
        bad = []
        for nm, p in self.net.named_parameters():
            if p.grad is not None and not torch.isfinite(p.grad).all():
                bad.append((nm, int((~torch.isfinite(p.grad)).sum())))
            if len(bad) >= 6:
                break
        print(f"step {self.step + 1}: non-finite grad_norm, step skipped; bad={bad}", flush=True)

    def _dump_nan_batch(self, latents, labels) -> None:
        if self._nan_dumped:
            return
        self._nan_dumped = True
        path = os.path.join(self.cfg.run.out_dir, f"nan_batch_r{self.rank}.pt")
        if not os.path.exists(path):
            os.makedirs(self.cfg.run.out_dir, exist_ok=True)
            torch.save({"latents": latents.cpu(), "labels": labels.cpu(), "step": self.step},
                       path)
            print(f"rank {self.rank}: dumped non-finite-loss batch to {path}", flush=True)

    def train_step(self, latents, labels=None, batches=None) -> Dict[str, float]:
        """One optimizer step.  ``batches``: optional iterable of
        (latents, labels) micro-batches for grad_accum > 1."""
        micro = list(batches) if batches is not None else [(latents, labels)]
        losses, parts = [], {}
        for i, (lat, lab) in enumerate(micro):
            if hasattr(self.grad_sync, "armed"):
                # gradient buckets may leave for their owners during the LAST backward only
                self.grad_sync.armed = i == len(micro) - 1
            loss, parts = self.micro_step(lat, lab)
            losses.append(loss)
        dt, dev = losses[0].dtype, losses[0].device
        as_t = lambda v: (v if torch.is_tensor(v) else torch.tensor(float(v))).to(dt).to(dev) \
            .reshape(())
        split = (self.cfg.run.overlap_stats_read and dev.type == "cuda"
                 and getattr(self.grad_sync, "handles_ema", False))
        if split:
            # The host waits for the losses, the gradient norm and the skip flag only: they
            # are copied to pinned memory BEFORE the update kernels are enqueued, so the
            # optimizer phase of this step still runs while the host returns and enqueues the
            # first (small, launch-bound) kernels of the next step.  The QK-clip statistics
            # and the kernel status word, which exist only after the update, are those of the
            # PREVIOUS step (``flush_stats`` returns the last ones).
            if self._early_host is None:
                self._early_host = torch.zeros(5, dtype=torch.float32).pin_memory()
                self._late_host = torch.zeros(3, dtype=torch.float32).pin_memory()
                self._early_ev, self._late_ev = torch.cuda.Event(), torch.cuda.Event()

            def early(grad_norm, skipped):
                v = torch.stack([torch.stack(losses).mean(), parts["loss_u"], parts["loss_v"],
                                 as_t(grad_norm), as_t(skipped)]).float()
                self._early_host.copy_(v, non_blocking=True)
                self._early_ev.record()

            stats = self.optimizer_step(early=early)
            if self._late_pending:
                self._late_ev.synchronize()          # long done: it is a step old
            prev_late = self._late_host.tolist() if self._late_pending else [0.0, 0.0, 0.0]
            late = torch.stack([as_t(stats["qk_hot"]), as_t(stats["qk_smax"]),
                                as_t(self._status_scalar())]).float()
            self._late_host.copy_(late, non_blocking=True)
            self._late_ev.record()
            self._late_pending = True
            self._early_ev.synchronize()
            vec = self._early_host.tolist() + prev_late
        else:
            stats = self.optimizer_step()
            # ONE device -> host read per step: losses, norm, skip flag, QK-clip statistics and
            # the kernel status word (a bounded wait that ran out inside any kernel of this step)
            vec = torch.stack([torch.stack(losses).mean(), parts["loss_u"], parts["loss_v"],
                               as_t(stats["grad_norm"]), as_t(stats["skipped"]),
                               as_t(stats["qk_hot"]), as_t(stats["qk_smax"]),
                               as_t(self._status_scalar())]).tolist()
        self._raise_on_status(int(vec[7]))
        if not math.isfinite(vec[0]):
            self._dump_nan_batch(parts["_latents"], parts["_labels"])
        skipped = bool(vec[4])
        if skipped:
            if hasattr(self.grad_sync, "undo_step_count"):
                self.grad_sync.undo_step_count()
                self._report_bad_grads()
        stats.update(loss=vec[0], loss_u=vec[1], loss_v=vec[2], grad_norm=vec[3], skipped=skipped,
                     qk_hot=int(vec[5]), qk_smax=vec[6])
        self.last = stats
        return stats

    def flush_stats(self) -> Dict[str, float]:
        """Waits for the last step's update kernels and returns its QK-clip statistics;
        raises if one of its kernels gave up on a bounded wait.  Only needed with
        ``run.overlap_stats_read`` (where ``train_step`` reports these one step late); call it
        after the last step and before trusting the weights (``save`` does)."""
        if not getattr(self, "_late_pending", False):
            return {}
        self._late_ev.synchronize()
        hot, smax, status = self._late_host.tolist()
        self._late_pending = False
        self._raise_on_status(int(status))
        return {"qk_hot": int(hot), "qk_smax": smax}

    def _status_scalar(self):
        """The device status word of this rank's GPU (0 on CPU or before any kernel ran)."""
        if self.device.type != "cuda":
            return 0.0
        try:
            from .ops import cuda as cu
            if not cu.available():
                return 0.0
            from .ops import kernels as K
        except Exception:
            return 0.0
        return K.status_word(self.device)[0]

    def _raise_on_status(self, code: int) -> None:
        """A kernel of this step gave up on a bounded wait (a peer rank that never
        arrived, a TMA load or MMA that never completed): its output is not valid, so
        the step must not be trusted.  The CUDA context itself stays usable."""
        if code == 0:
            return
        from .ops import kernels as K

        K.status_word(self.device).zero_()
        raise RuntimeError(
            f"rank {self.rank}: imf_b200 kernel status {code} "
            f"({K.STATUS_NAMES.get(code, 'unknown')}) at step {self.step}; gradients or "
            "weights of this step are not valid on this rank")

    # -------------------------------------------------------- checkpoints --
    def save(self, path: Optional[str] = None, sampler_state: Optional[Dict[str, int]] = None
             ) -> Optional[str]:
        """Collective: every rank calls it.  Rank 0 writes; all ranks leave together, so no
        rank runs ahead into the next step's peer barrier while rank 0 is still in fsync.
        ``extra`` carries the RNG state, the world size, the Muon owner map and the
        sampler position (epoch, batches consumed) for an exact resume."""
        self.flush_stats()       # a pending kernel status of the last step raises here
        extra: Dict[str, Any] = {"rng": ckpt_mod.rng_state(), "world": self.world}
        if hasattr(self.grad_sync, "owner_table"):
            extra["muon_owner"] = list(self.grad_sync.owner_table())
        if sampler_state:
            extra["sampler"] = {k: int(v) for k, v in sampler_state.items()}
        if hasattr(self.grad_sync, "gather_state"):
            self.grad_sync.gather_state()     # collective: every rank calls save()
        out = None
        if self.rank == 0:
            out = path or ckpt_mod.checkpoint_path(self.cfg.run.out_dir, self.step)
            ckpt_mod.save_checkpoint(out, self.net, self.optimizer, self.ema, self.step,
                                     config_as_dict(self.cfg), extra)
            if self.verbose:
                print(f"saved {out}", flush=True)
        if self.world > 1:
            pdist.barrier()
        return out

    def load(self, path: str, restore_rng: bool = False) -> None:
        info = ckpt_mod.load_checkpoint(path, self.net, self.optimizer, self.ema, self.rank,
                                        self.world, barrier=pdist.barrier)
        self.step = info["step"]
        extra = info.get("extra", {}) or {}
        saved_owner = extra.get("muon_owner")
        if saved_owner is not None and hasattr(self.grad_sync, "owner_table") \
                and extra.get("world") == self.world \
                and list(saved_owner) != list(self.grad_sync.owner_table()):
            raise RuntimeError("checkpoint was written with a different Muon owner map for the "
                               "same world size; momentum segments would not line up")
        self.resume_sampler = extra.get("sampler")
        if restore_rng and "rng" in info.get("extra", {}) and self.world == 1:
            ckpt_mod.set_rng_state(info["extra"]["rng"])
        if hasattr(self.grad_sync, "after_load"):
            self.grad_sync.after_load()
        if self.verbose:
            print(f"resumed from {path} at step {self.step}", flush=True)


# ------------------------------------------------------------------ main ---
def main(argv=None) -> None:
    cfg = config_mod.parse_cli(sys.argv[1:] if argv is None else argv)
    rank, world, _local, device = pdist.init_distributed()
    trainer = Trainer(cfg, rank, world, device)
    _ds, sampler, loader = build_loader(cfg.data, cfg.model, rank, world,
                                        device.type == "cuda", seed=cfg.run.seed)
    if cfg.run.resume:
        trainer.load(cfg.run.resume)
    hb = None
    if world > 1 and cfg.run.heartbeat_s > 0:
        store = dist.distributed_c10d._get_default_store()
        hb = pdist.Heartbeat(store, rank, world, period_s=cfg.run.heartbeat_s,
                             stale_s=10 * cfg.run.heartbeat_s).start()
    use_wandb = bool(cfg.run.wandb_project) and rank == 0
    if use_wandb:
        import wandb

        wandb.init(project=cfg.run.wandb_project, config=config_as_dict(cfg))
    os.makedirs(cfg.run.out_dir, exist_ok=True)
    inf = InfiniteLoader(loader, sampler)
    if cfg.run.resume and getattr(trainer, "resume_sampler", None):
        inf.restore(trainer.resume_sampler)
    batches = DevicePrefetcher(inf, device)
    o = cfg.optim
    loss_u_ema, t_log = None, time.time()
    while trainer.step < o.total_steps:
        if hb is not None:
            hb.check()
        micro = [next(batches) for _ in range(o.grad_accum)]
        st = trainer.train_step(None, batches=micro)
        step = trainer.step
        if rank == 0 and step % cfg.run.log_every == 0:
            dt = time.time() - t_log
            sps = cfg.run.log_every * cfg.data.batch_size_per_gpu * world * o.grad_accum / dt
            lu = st["loss_u"]
            if loss_u_ema is None:
                loss_u_ema = lu
            elif math.isfinite(lu):
                loss_u_ema = 0.8 * loss_u_ema + 0.2 * lu
            print(f"step {step} loss={st['loss']:.4f} loss_u={lu:.4f} "
                  f"loss_u_ema={loss_u_ema:.4f} loss_v={st['loss_v']:.4f} "
                  f"grad_norm={st['grad_norm']:.3f} lr={st['lr']:.2e} "
                  f"qkclip={st['qk_hot']}/{st['qk_smax']:.0f} {sps:.1f} samples/s", flush=True)
            if cfg.run.profile_phases:
                ms = PhaseTimer.reduce_max(trainer.timer.summary())
                print("  phases(ms, max over ranks): "
                      + " ".join(f"{k}={v:.1f}" for k, v in sorted(ms.items())), flush=True)
            if use_wandb:
                wandb.log({"loss": st["loss"], "grad_norm": st["grad_norm"], "lr": st["lr"],
                           "samples_per_s": sps}, step=step)
            t_log = time.time()
        if step % cfg.run.ckpt_every == 0:
            trainer.save(sampler_state=inf.state(prefetched=1))
    trainer.flush_stats()        # the last step's kernel status word (raises if one gave up)
    if hb is not None:
        hb.stop()
    pdist.shutdown()


if __name__ == "__main__":
    main()
