"""improved-MeanFlow training objective and sampler for video latents.

Same sampling laws, guidance rule, adaptive weighting and public API as the
reference ``IMFVideoLoss`` (``imf_video.py:16-657``).  What differs is how the
three quantities (u, du/dt, v) are obtained: the default path evaluates the
network ONCE on dual numbers (``IMFDiTVideo.forward_dual``), and the
guidance passes run only the trunk + v branch.  The reference runs the u
branch in the guidance passes and throws it away (``imf_video.py:326``), and
computes the primal u twice (``imf_video.py:506-522``).
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from .ops.dual import Dual

Tensor = torch.Tensor


class IMFVideoLoss(nn.Module):
    def __init__(self, net, num_classes, P_mean=-0.4, P_std=1.0, data_proportion=0.5,
                 cfg_beta=1.0, class_dropout_prob=0.1, s_max=7.0, norm_p=1.0, norm_eps=0.01,
                 loss_v_weight=1.0, jvp_impl="fused", stratified_time=True,
                 stratified_interval=False, strat_group=0, autocast_bf16=False,
                 reuse_ungated_guidance=False):
        super().__init__()
        assert jvp_impl in ("fused", "fast", "functorch")
        assert not (autocast_bf16 and jvp_impl == "functorch"), \
            "autocast_bf16 needs the fused dual-number path"
        self.net = net
        self.num_classes = num_classes
        self.P_mean, self.P_std = P_mean, P_std
        self.data_proportion = data_proportion
        self.cfg_beta, self.s_max = cfg_beta, s_max
        self.class_dropout_prob = class_dropout_prob
        self.norm_p, self.norm_eps = norm_p, norm_eps
        self.loss_v_weight = loss_v_weight
        self.jvp_impl = jvp_impl
        self.stratified_time = stratified_time
        self.stratified_interval = stratified_interval
        self.strat_group = strat_group
        self.autocast_bf16 = autocast_bf16
        # skip the second (interval-gated) guidance pass for samples whose gate
        # left omega unchanged: the result is identical, one host sync per step
        self.reuse_ungated_guidance = reuse_ungated_guidance
        self._strat_queues: Dict[str, Tensor] = {}
        if autocast_bf16 and getattr(net, "compute_dtype", None) is None:
            net.compute_dtype = torch.bfloat16

    # ---------------------------------------------------------- sampling ---
    def _take_strata(self, bz: int, device, site: str) -> Tensor:
        """Pop ``bz`` stratum indices from ``site``'s reshuffled 0..G-1 queue
        so G consecutive draws (over several micro-batches) cover each stratum
        once (reference ``imf_video.py:91-115``)."""
        g = self.strat_group
        q = self._strat_queues.get(site)
        while q is None or q.numel() < bz:
            fresh = torch.randperm(g, device=device)
            q = fresh if q is None else torch.cat([q, fresh])
        self._strat_queues[site] = q[bz:]
        return q[:bz].to(torch.float32)

    def _strat_uniform(self, bz: int, device, site: str = "default") -> Tensor:
        """Jittered-quantile U(0,1) draws, one per equal-probability stratum."""
        if not self.stratified_time:
            return torch.rand(bz, device=device, dtype=torch.float32)
        if self.strat_group and self.strat_group > bz:
            i, g = self._take_strata(bz, device, site), self.strat_group
        else:
            i, g = torch.randperm(bz, device=device).to(torch.float32), bz
        u = (i + torch.rand(bz, device=device)) / g
        return u.clamp(1e-6, 1 - 1e-6)

    def logit_normal_dist(self, bz, device, dtype, site="time") -> Tensor:
        if self.stratified_time:
            u = self._strat_uniform(bz, device, site)
            z = (torch.erfinv(2 * u - 1) * math.sqrt(2.0)).reshape(bz, 1, 1, 1, 1).to(dtype)
        else:
            z = torch.randn(bz, 1, 1, 1, 1, device=device, dtype=dtype)
        return torch.sigmoid(z * self.P_std + self.P_mean)

    def sample_tr(self, bz, device, dtype):
        """t >= r logit-normal; a ``data_proportion`` share (stratified) is
        forced to r = t, i.e. plain flow matching."""
        a = self.logit_normal_dist(bz, device, dtype, "time_t")
        b = self.logit_normal_dist(bz, device, dtype, "time_r")
        t, r = torch.maximum(a, b), torch.minimum(a, b)
        fm_mask = (self._strat_uniform(bz, device, "fm_split") < self.data_proportion
                   ).reshape(bz, 1, 1, 1, 1)
        return t, torch.where(fm_mask, t, r), fm_mask

    def sample_cfg_scale(self, bz, device) -> Tensor:
        """omega in [1, 1 + s_max] with density tilted by ``cfg_beta``."""
        u = self._strat_uniform(bz, device, "omega").reshape(bz, 1, 1, 1, 1)
        top = math.log1p(self.s_max)
        if self.cfg_beta == 1.0:
            return torch.exp(u * top).float()
        e = 1.0 - self.cfg_beta
        return torch.exp(torch.log1p(u * math.expm1(e * top)) / e).float()

    def sample_cfg_interval(self, bz, device, dtype, fm_mask):
        if self.stratified_interval:
            lo = self._strat_uniform(bz, device, "t_min").reshape(bz, 1, 1, 1, 1).to(dtype)
            hi = self._strat_uniform(bz, device, "t_max").reshape(bz, 1, 1, 1, 1).to(dtype)
        else:
            lo = torch.rand(bz, 1, 1, 1, 1, device=device, dtype=dtype)
            hi = torch.rand(bz, 1, 1, 1, 1, device=device, dtype=dtype)
        t_min = torch.where(fm_mask, torch.zeros_like(lo), 0.5 * lo)
        t_max = torch.where(fm_mask, torch.ones_like(hi), 0.5 + 0.5 * hi)
        return t_min, t_max

    # ------------------------------------------------------ network calls ---
    @staticmethod
    def _flat(s: Tensor) -> Tensor:
        return s.reshape(s.shape[0])

    def u_fn(self, x, t, h, omega, t_min, t_max, y):
        """(u, v) through the network's reference-compatible entry."""
        f = self._flat
        u, v = self.net(x, f(t), f(h), f(omega), f(t_min), f(t_max), y)
        return u.float(), v.float()

    def _v_only(self, x, t, omega, y) -> Tensor:
        """v-head read with dummy h = 0 and interval [0, 1]; only the trunk and
        the v branch are evaluated."""
        f = self._flat
        net = self.net
        if hasattr(net, "forward_dual"):
            out = net.forward_dual(Dual(x), Dual(torch.zeros_like(f(t))), f(omega),
                                   torch.zeros_like(f(t)), torch.ones_like(f(t)), y,
                                   branches=("v",) if len(net.v_heads) else ("u",))
            return next(iter(out.values())).p.float()
        z = torch.zeros_like(t)
        return self.u_fn(x, t, z, omega, z, torch.ones_like(t), y)[1]

    def v_cond_fn(self, x, t, omega, y) -> Tensor:
        return self._v_only(x, t, omega, y)

    def v_fn(self, x, t, omega, y):
        """Conditional and null-label v in one 2B batch."""
        bz = x.shape[0]
        y_null = torch.full((bz,), self.num_classes, device=y.device, dtype=y.dtype)
        out = self._v_only(torch.cat([x, x]), torch.cat([t, t]),
                           torch.cat([omega, torch.ones_like(omega)]), torch.cat([y, y_null]))
        return out[:bz], out[bz:]

    def cond_drop(self, v_t, v_g, labels):
        """#drops ~ Binomial(B, p), applied to the LEADING samples (reference
        ``imf_video.py:359-395``); dropped samples take v_t as their target."""
        bz = v_t.shape[0]
        n = (torch.rand(bz, device=v_t.device) < self.class_dropout_prob).sum()
        drop = torch.arange(bz, device=v_t.device) < n
        labels = torch.where(drop, torch.full_like(labels, self.num_classes), labels)
        return labels, torch.where(drop.reshape(bz, 1, 1, 1, 1), v_t, v_g)

    def guidance_fn(self, v_t, z_t, t, r, y, fm_mask, w, t_min, t_max):
        """v_g = v_t + (1 - 1/w)(v_c - v_u); w -> 1 outside [t_min, t_max] for
        mean-flow samples; flow-matching samples use the ungated w."""
        v_c0, v_u = self.v_fn(z_t, t, w, y)
        v_g_fm = v_t + (1 - 1 / w) * (v_c0 - v_u)
        inside = (t >= t_min) & (t <= t_max)
        wg = torch.where(inside, w, torch.ones_like(w))
        if self.reuse_ungated_guidance:
            changed = self._flat(wg != w)
            if bool(changed.any()):
                if bool(changed.all()):
                    v_c = self.v_cond_fn(z_t, t, wg, y)
                else:
                    idx = changed.nonzero().squeeze(1)
                    v_c = v_c0.clone()
                    v_c[idx] = self.v_cond_fn(z_t[idx], t[idx], wg[idx], y[idx])
            else:
                v_c = v_c0
        else:
            v_c = self.v_cond_fn(z_t, t, wg, y)
        v_g = v_t + (1 - 1 / wg) * (v_c - v_u)
        return torch.where(fm_mask, v_g_fm, v_g), v_c

    # ------------------------------------------------------------ forward ---
    def _adaptive(self, per_sample: Tensor) -> Tensor:
        return per_sample / ((per_sample + self.norm_eps) ** self.norm_p).detach()

    def u_du_v(self, z_t, t, r, omega, t_min, t_max, labels, v_c):
        """u (graph), du/dt along (v_c, 1, 0) (detached), v (graph)."""
        f = self._flat
        if self.jvp_impl == "functorch":
            def fn(z, tt, rr):
                return self.u_fn(z, tt, tt - rr, omega, t_min, t_max, labels)
            u, du, v = torch.func.jvp(fn, (z_t, t, r),
                                      (v_c, torch.ones_like(t), torch.zeros_like(t)),
                                      has_aux=True)
            return u, du.detach(), v
        h = f(t - r)
        out = self.net.forward_dual(Dual(z_t, v_c.detach()), Dual(h, torch.ones_like(h)),
                                    f(omega), f(t_min), f(t_max), labels,
                                    branches=("u", "v"), tangent_branches=("u",))
        u = out["u"]
        v = out["v"].p if "v" in out else u.p
        du = u.t if u.t is not None else torch.zeros_like(u.p)
        return u.p.float(), du.float().detach(), v.float()

    def forward(self, latents: Tensor, labels: Tensor):
        x = latents
        bz, device, dtype = x.shape[0], x.device, x.dtype
        t, r, fm_mask = self.sample_tr(bz, device, dtype)
        e = torch.randn_like(x)
        z_t = (1 - t) * x + t * e
        v_t = e - x
        t_min, t_max = self.sample_cfg_interval(bz, device, dtype, fm_mask)
        omega = self.sample_cfg_scale(bz, device)

        with torch.no_grad():
            v_g, v_c = self.guidance_fn(v_t, z_t, t, r, labels, fm_mask, omega, t_min, t_max)
        labels, v_g = self.cond_drop(v_t, v_g, labels)

        u, du_dt, v = self.u_du_v(z_t, t, r, omega, t_min, t_max, labels, v_c)
        V = u + (t - r) * du_dt.detach()
        v_g = v_g.detach()
        err_u, err_v = (V - v_g) ** 2, (v - v_g) ** 2
        loss_u = self._adaptive(err_u.sum(dim=(1, 2, 3, 4)))
        loss_v = self._adaptive(err_v.sum(dim=(1, 2, 3, 4)))
        loss = (loss_u + self.loss_v_weight * loss_v).mean()
        return loss, {"loss": loss.detach(), "loss_u": err_u.mean().detach(),
                      "loss_v": err_v.mean().detach()}

    # ------------------------------------------------------------ sampler ---
    @torch.no_grad()
    def sample_one_step(self, z_t, labels, t, r, omega, t_min, t_max):
        """z_r = z_t - (t - r) u(z_t, t, t - r)."""
        f = self._flat
        net = self.net
        if hasattr(net, "forward_dual"):
            u = net.forward_dual(Dual(z_t), Dual(f(t - r)), f(omega), f(t_min), f(t_max),
                                 labels, branches=("u",))["u"].p.float()
        else:
            u = self.u_fn(z_t, t, t - r, omega, t_min, t_max, labels)[0]
        return z_t - (t - r) * u.to(z_t.dtype)

    @torch.no_grad()
    def sample(self, z_1, labels, num_steps=None, omega=None, t_min=None, t_max=None,
               t_steps=None):
        """Integrate from t = 1 (noise) to t = 0 in ``num_steps`` mean-flow
        steps; defaults come from ``config.sample``."""
        from .config import config as _cfg

        s = _cfg.sample
        num_steps = s.num_steps if num_steps is None else num_steps
        omega = s.omega if omega is None else omega
        t_min = s.t_min if t_min is None else t_min
        t_max = s.t_max if t_max is None else t_max
        device, dtype, bz = z_1.device, z_1.dtype, z_1.shape[0]
        if t_steps is None:
            t_steps = torch.linspace(1.0, 0.0, num_steps + 1, device=device, dtype=dtype)
        else:
            t_steps = torch.as_tensor(t_steps, device=device, dtype=dtype)
        full = lambda val: torch.full((bz, 1, 1, 1, 1), float(val), device=device, dtype=dtype)
        om, lo, hi = full(omega), full(t_min), full(t_max)
        z = z_1
        for i in range(t_steps.shape[0] - 1):
            z = self.sample_one_step(z, labels, full(t_steps[i]), full(t_steps[i + 1]),
                                     om, lo, hi)
        return z
