"""Moonlight = Muon (momentum -> quintic Newton-Schulz -> RMS-matched step,
decoupled weight decay) on hidden matrices + AdamW on everything else.

Math, hyper-parameters, parameter routing and per-parameter state keys
(``momentum_buffer`` / ``step, exp_avg, exp_avg_sq``) match the reference
optimizer (``moonlight.py:203-540``) so optimizer state dicts interchange.
The execution differs:

* matrices of the same (n, m) are stacked and orthogonalised together (one
  batched Newton-Schulz per shape instead of a Python loop per parameter,
  reference ``moonlight.py:395-437``);
* with ``owner_map`` (see ``parallel/owner.py``) each rank runs Newton-Schulz
  only for the matrices it owns and the others receive the result, instead of
  every rank repeating all of it;
* the AdamW branch runs as a multi-tensor (foreach) update.
"""

from __future__ import annotations

import json
import math
import os
from collections import defaultdict
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

Tensor = torch.Tensor

JORDAN_COEFFS = (3.4445, -4.7750, 2.0315)
_COEFF_CACHE: Dict[Tuple[int, int, int], Tuple[float, float, float]] = {}
_PACKAGED_CACHE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ns_coeffs.json")


# ----------------------------------------------------- coefficient solve ---
def sample_normalized_spectrum(n, m, num_samples=32, seed=0, device="cpu") -> Tensor:
    """Singular values of ``num_samples`` Gaussian (n, m) matrices, each set
    divided by its Frobenius norm (what Newton-Schulz sees after X/||X||_F)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    vals = []
    for _ in range(num_samples):
        s = torch.linalg.svdvals(torch.randn(n, m, generator=g, dtype=torch.float32).to(device))
        vals.append(s / s.norm())
    return torch.cat(vals)


def _iterate_scalar(x: Tensor, kappa, x1, x2, steps: int) -> Tensor:
    for _ in range(steps):
        x = x + kappa * x * (x * x - x1 * x1) * (x * x - x2 * x2)
    return x


def solve_ns_coefficients(n, m, steps=5, num_samples=32, opt_iters=3000, lr=2e-2, seed=0,
                          device="cpu"):
    """Fit the quintic g(x) = x + k x (x^2 - x1^2)(x^2 - x2^2) so that ``steps``
    applications map the shape's normalised spectrum to 1 (Su Jianlin's
    fixed-point parameterisation, as in reference ``moonlight.py:86-146``).
    Returns ((a, b, c), mse) with a = 1 + k x1^2 x2^2, b = -k (x1^2 + x2^2),
    c = k."""
    sigma = sample_normalized_spectrum(n, m, num_samples, seed, device)
    theta = torch.tensor([1.0, 0.9, 1.1], device=sigma.device, requires_grad=True)
    opt = torch.optim.Adam([theta], lr=lr)
    for _ in range(opt_iters):
        opt.zero_grad()
        loss = (_iterate_scalar(sigma, theta[0], theta[1], theta[2], steps) - 1).pow(2).mean()
        loss.backward()
        opt.step()
    with torch.no_grad():
        k, x1, x2 = (float(z) for z in theta)
        mse = float((_iterate_scalar(sigma, k, x1, x2, steps) - 1).pow(2).mean())
    return (1.0 + k * x1 * x1 * x2 * x2, -k * (x1 * x1 + x2 * x2), k), mse


def _disk_paths() -> List[str]:
    paths = []
    env = os.environ.get("MOONLIGHT_COEFF_CACHE")
    if env:
        paths.append(env)
    paths.append(_PACKAGED_CACHE)
    return paths


def get_ns_coefficients(n, m, steps, mode="per_shape", verbose=False, **solve_kw):
    """(a, b, c) for a shape; solved once per (min, max, steps) and cached in
    memory and on disk (``MOONLIGHT_COEFF_CACHE`` JSON, then the packaged
    table).  Keys are ``"{min}x{max}x{steps}"`` as in the reference's cache."""
    if mode == "jordan":
        return JORDAN_COEFFS
    if mode != "per_shape":
        raise ValueError(f"unknown coefficient mode {mode!r}")
    n, m = min(n, m), max(n, m)
    key = (n, m, steps)
    if key in _COEFF_CACHE:
        return _COEFF_CACHE[key]
    skey = f"{n}x{m}x{steps}"
    for path in _disk_paths():
        if os.path.exists(path):
            try:
                with open(path) as fh:
                    disk = json.load(fh)
            except (OSError, ValueError):
                continue
            if skey in disk:
                _COEFF_CACHE[key] = tuple(disk[skey])
                return _COEFF_CACHE[key]
    coeffs, mse = solve_ns_coefficients(n, m, steps=steps, **solve_kw)
    _COEFF_CACHE[key] = coeffs
    env = os.environ.get("MOONLIGHT_COEFF_CACHE")
    if env:
        disk = {}
        if os.path.exists(env):
            try:
                with open(env) as fh:
                    disk = json.load(fh)
            except (OSError, ValueError):
                disk = {}
        disk[skey] = list(coeffs)
        tmp = env + ".tmp"
        with open(tmp, "w") as fh:
            json.dump(disk, fh, indent=1)
        os.replace(tmp, env)
    if verbose:
        print(f"  NS coeffs ({n:>5},{m:>5}) T={steps}: a={coeffs[0]:+.4f} "
              f"b={coeffs[1]:+.4f} c={coeffs[2]:+.4f} mse={mse:.3e}")
    return coeffs


# ------------------------------------------------------- Newton-Schulz -----
def zeropower_via_newtonschulz5(G: Tensor, steps=5, eps=1e-7, dtype=None, coeffs=None,
                                out: Optional[Tensor] = None) -> Tensor:
    """Approximate U V^T of G = U S V^T.  Accepts (n, m) or a batch (k, n, m).
    X = G / (||G||_F + eps); transposed when n > m so the Gram matrix is the
    small one; ``steps`` x {A = X X^T; B = bA + cA^2; X = aX + BX}.
    bf16 on CUDA, fp32 elsewhere (reference ``moonlight.py:203-252``)."""
    assert G.ndim in (2, 3), f"Newton-Schulz needs matrices, got {tuple(G.shape)}"
    a, b, c = JORDAN_COEFFS if coeffs is None else coeffs
    if dtype is None:
        dtype = torch.bfloat16 if G.is_cuda else torch.float32
    if G.is_cuda and G.ndim == 3:
        from ..ops import cuda as cu

        if cu.available() and cu.has("newton_schulz") and dtype == torch.bfloat16:
            res = cu.newton_schulz(G, (a, b, c), steps, eps, out=out)
            if res is not None:
                return res
    X = G.to(dtype)
    nrm = X.flatten(-2).norm(dim=-1)
    X = X / (nrm.reshape(nrm.shape + (1, 1)) + eps)
    tr = G.shape[-2] > G.shape[-1]
    if tr:
        X = X.transpose(-1, -2)
    for _ in range(steps):
        A = X @ X.transpose(-1, -2)
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    X = X.transpose(-1, -2) if tr else X
    if out is not None:
        out.copy_(X)
        return out
    return X


# ----------------------------------------------------------- optimizer -----
class Moonlight(torch.optim.Optimizer):
    """Param groups carry ``use_muon``; both branches honour ``group["lr"]``.

    ``owner_of``: optional ``param -> rank`` map; with ``rank``/``world`` and
    ``exchange`` set (see ``parallel.owner.attach``) only owned matrices are
    orthogonalised locally."""

    def __init__(self, muon_params=None, adamw_params=None, lr=1e-3, weight_decay=0.1,
                 momentum=0.95, nesterov=True, ns_steps=5, lr_scale_constant=0.2,
                 adamw_betas=(0.9, 0.95), adamw_eps=1e-8, ns_dtype=None,
                 coeff_mode="per_shape", coeff_samples=32, coeff_iters=3000, coeff_lr=2e-2,
                 coeff_seed=0, verbose=False):
        muon_params = list(muon_params or [])
        adamw_params = list(adamw_params or [])
        assert muon_params or adamw_params, "no parameters given"
        for p in muon_params:
            assert p.ndim >= 2, (f"Muon needs matrices, got shape {tuple(p.shape)}; "
                                 "route it to adamw_params")
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov,
                        ns_steps=ns_steps, lr_scale_constant=lr_scale_constant,
                        adamw_betas=adamw_betas, adamw_eps=adamw_eps, ns_dtype=ns_dtype,
                        coeff_mode=coeff_mode)
        groups = []
        if muon_params:
            groups.append({"params": muon_params, "use_muon": True})
        if adamw_params:
            groups.append({"params": adamw_params, "use_muon": False})
        super().__init__(groups, defaults)
        self._solve_kw = dict(num_samples=coeff_samples, opt_iters=coeff_iters, lr=coeff_lr,
                              seed=coeff_seed)
        self.distributed = None        # set by parallel.owner.attach
        if coeff_mode == "per_shape" and muon_params:
            shapes = sorted({self._matrix_shape(p) for p in muon_params})
            if verbose:
                print(f"Moonlight: Newton-Schulz coefficients for {len(shapes)} shapes "
                      f"(steps={ns_steps})")
            for shp in shapes:
                get_ns_coefficients(*shp, steps=ns_steps, mode=coeff_mode, verbose=verbose,
                                    **self._solve_kw)

    @staticmethod
    def _matrix_shape(p) -> Tuple[int, int]:
        return (p.shape[0], p.numel() // p.shape[0]) if p.ndim > 2 else tuple(p.shape)

    @staticmethod
    def muon_lr_scale(matrix_shape, constant) -> float:
        """constant * sqrt(max(n, m)): pins the update RMS at ``constant``."""
        return constant * math.sqrt(max(matrix_shape))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self.distributed is not None:
            self.distributed.step(self)
            return loss
        for group in self.param_groups:
            if group["use_muon"]:
                self._muon_step(group)
            else:
                self._adamw_step(group)
        return loss

    # -- Muon ----------------------------------------------------------------
    def _muon_direction(self, group, p) -> Tensor:
        """Momentum update; returns the (n, m) matrix handed to Newton-Schulz."""
        g = p.grad.reshape(p.grad.shape[0], -1) if p.grad.ndim > 2 else p.grad
        st = self.state[p]
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros_like(g)
        buf = st["momentum_buffer"]
        buf.mul_(group["momentum"]).add_(g)
        return g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf

    def _orthogonalize(self, group, mats: Sequence[Tensor]) -> List[Tensor]:
        """Newton-Schulz on a list of matrices, batched per shape."""
        by_shape: Dict[Tuple[int, int], List[int]] = defaultdict(list)
        for i, mtx in enumerate(mats):
            by_shape[tuple(mtx.shape)].append(i)
        out: List[Optional[Tensor]] = [None] * len(mats)
        for shp, idxs in by_shape.items():
            coeffs = get_ns_coefficients(*shp, steps=group["ns_steps"],
                                         mode=group["coeff_mode"], **self._solve_kw)
            stack = torch.stack([mats[i] for i in idxs])
            upd = zeropower_via_newtonschulz5(stack, steps=group["ns_steps"],
                                              dtype=group["ns_dtype"], coeffs=coeffs)
            for j, i in enumerate(idxs):
                out[i] = upd[j]
        return out  # type: ignore[return-value]

    def _muon_apply(self, group, p, update: Tensor) -> None:
        lr, wd = group["lr"], group["weight_decay"]
        scale = self.muon_lr_scale(tuple(update.shape), group["lr_scale_constant"])
        p.mul_(1 - lr * wd)
        p.add_(update.reshape(p.shape).to(p.dtype), alpha=-lr * scale)

    def _muon_step(self, group) -> None:
        params = [p for p in group["params"] if p.grad is not None]
        if not params:
            return
        dirs = [self._muon_direction(group, p) for p in params]
        for p, u in zip(params, self._orthogonalize(group, dirs)):
            self._muon_apply(group, p, u)

    # -- AdamW ---------------------------------------------------------------
    def _adamw_step(self, group) -> None:
        """Textbook bias-corrected AdamW with decoupled weight decay; state
        ``step`` is a Python int as in the reference (``moonlight.py:439-469``)."""
        lr, wd = group["lr"], group["weight_decay"]
        b1, b2 = group["adamw_betas"]
        eps = group["adamw_eps"]
        by_step: Dict[int, List[Tensor]] = defaultdict(list)
        for p in group["params"]:
            if p.grad is None:
                continue
            st = self.state[p]
            if "step" not in st:
                st["step"] = 0
                st["exp_avg"] = torch.zeros_like(p)
                st["exp_avg_sq"] = torch.zeros_like(p)
            st["step"] += 1
            by_step[st["step"]].append(p)
        for t, ps in by_step.items():
            gs = [p.grad for p in ps]
            m = [self.state[p]["exp_avg"] for p in ps]
            v = [self.state[p]["exp_avg_sq"] for p in ps]
            torch._foreach_mul_(m, b1)
            torch._foreach_add_(m, gs, alpha=1 - b1)
            torch._foreach_mul_(v, b2)
            torch._foreach_addcmul_(v, gs, gs, value=1 - b2)
            bias1, bias2 = 1 - b1 ** t, 1 - b2 ** t
            den = torch._foreach_div(v, bias2)
            torch._foreach_sqrt_(den)
            torch._foreach_add_(den, eps)
            torch._foreach_mul_(ps, 1 - lr * wd)
            torch._foreach_addcdiv_(ps, m, den, value=-lr / bias1)


ADAMW_NAME_MARKERS = ("embedding_table", "_tokens", "_embedder", "x_embedder", "final_layer",
                      "alpha_logit")


def is_adamw_param(name: str, p: Tensor) -> bool:
    """AdamW takes every <2-D parameter, embeddings, token banks, the scalar
    embedders, the patch embed, the output layers and the SLA2 mixing logits;
    Muon takes the remaining matrices (incl. Linear(d,1) score heads, router
    projections and g_proj) -- reference ``moonlight.py:472-540``."""
    return p.ndim < 2 or any(mk in name for mk in ADAMW_NAME_MARKERS)


def split_params(model, verbose=False):
    muon, adamw = [], []
    for name, p in model.named_parameters():
        if p.requires_grad:
            (adamw if is_adamw_param(name, p) else muon).append(p)
    total = sum(p.numel() for p in model.parameters() if p.requires_grad)
    nm, na = sum(p.numel() for p in muon), sum(p.numel() for p in adamw)
    assert nm + na == total
    if verbose:
        print(f"Moonlight split: Muon {len(muon)} tensors / {nm / 1e6:.1f}M params, "
              f"AdamW {len(adamw)} tensors / {na / 1e6:.1f}M params")
    return muon, adamw


def build_moonlight(model, lr, weight_decay, momentum=0.95, nesterov=True, ns_steps=5,
                    lr_scale_constant=0.2, adamw_betas=(0.9, 0.95), adamw_eps=1e-8,
                    coeff_mode="per_shape", coeff_samples=32, coeff_iters=3000, coeff_lr=2e-2,
                    coeff_seed=0, verbose=False) -> Moonlight:
    muon, adamw = split_params(model, verbose=verbose)
    return Moonlight(muon, adamw, lr=lr, weight_decay=weight_decay, momentum=momentum,
                     nesterov=nesterov, ns_steps=ns_steps, lr_scale_constant=lr_scale_constant,
                     adamw_betas=adamw_betas, adamw_eps=adamw_eps, coeff_mode=coeff_mode,
                     coeff_samples=coeff_samples, coeff_iters=coeff_iters, coeff_lr=coeff_lr,
                     coeff_seed=coeff_seed, verbose=verbose)
