"""Plain-PyTorch formulas for every dual-number (primal, tangent) op.

These are the CPU path, the oracle for every CUDA kernel test, and the
numerics contract of the framework.  Each ``*_jvp`` function returns
``(y, dy)`` for inputs ``(x, dx)``; parameters carry no tangent (the iMF
loss differentiates w.r.t. time only, reference ``imf_video.py:485-533``).

All math is done in fp32 regardless of the storage dtype, matching the
reference modules (``models/imf_dit_video.py:121-165``, ``:266-320``).
"""

from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

Tensor = torch.Tensor


# --------------------------------------------------------------------------
# RMSNorm
# --------------------------------------------------------------------------
def rmsnorm(x: Tensor, weight: Optional[Tensor], eps: float) -> Tensor:
    xf = x.float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * r).to(x.dtype)
    return y if weight is None else y * weight


def rmsnorm_jvp(x: Tensor, dx: Tensor, weight: Optional[Tensor], eps: float
                ) -> Tuple[Tensor, Tensor]:
    """y = x r g with r = rsqrt(mean x^2 + eps);
    dy = g (r dx - x r^3 mean(x dx))."""
    xf, dxf = x.float(), dx.float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = xf * r
    dy = dxf * r - xf * (r.pow(3) * (xf * dxf).mean(-1, keepdim=True))
    if weight is not None:
        w = weight.float()
        y, dy = y * w, dy * w
    return y.to(x.dtype), dy.to(dx.dtype)


# --------------------------------------------------------------------------
# SituAndMul: beta tanh(g/beta) sigmoid(g) * (lbeta tanh(up/lbeta))
# --------------------------------------------------------------------------
def situ_mul(gate: Tensor, up: Tensor, beta: float,
             linear_beta: Optional[float]) -> Tensor:
    g, u = gate.float(), up.float()
    a = beta * torch.tanh(g / beta) * torch.sigmoid(g)
    if linear_beta is not None:
        u = linear_beta * torch.tanh(u / linear_beta)
    return (a * u).to(gate.dtype)


def situ_mul_jvp(gate: Tensor, up: Tensor, dgate: Tensor, dup: Tensor,
                 beta: float, linear_beta: Optional[float]
                 ) -> Tuple[Tensor, Tensor]:
    """Includes the ``linear_beta`` clamp on the up branch in the tangent
    (the reference's Triton tangent kernel omits it,
    ``models/triton_mla_block_jvp.py:437-471``; the module applies it,
    ``models/imf_dit_video.py:163-164``)."""
    g, u = gate.float(), up.float()
    dg, du = dgate.float(), dup.float()
    th = torch.tanh(g / beta)
    sg = torch.sigmoid(g)
    a = beta * th * sg
    da = ((1 - th * th) * sg + beta * th * sg * (1 - sg)) * dg
    if linear_beta is not None:
        tu = torch.tanh(u / linear_beta)
        du = (1 - tu * tu) * du
        u = linear_beta * tu
    return (a * u).to(gate.dtype), (da * u + a * du).to(dgate.dtype)


# --------------------------------------------------------------------------
# Rotary embedding on adjacent (even, odd) channel pairs
# --------------------------------------------------------------------------
def rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """x: (b, l, H, dr); cos/sin: (l, dr/2). Linear in x, so the tangent of
    rope(x) is rope(dx)."""
    xf = x.float()
    xr, xi = xf[..., 0::2], xf[..., 1::2]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    out = torch.stack([xr * c - xi * s, xr * s + xi * c], dim=-1).flatten(-2)
    return out.to(x.dtype)


# --------------------------------------------------------------------------
# Dense attention (b, l, H, d) layout, softmax scale 1/sqrt(dk)
# --------------------------------------------------------------------------
def _q_chunk(l: int, s: int, bh: int, budget_bytes: int = 1 << 30) -> int:
    per_row = max(1, s * bh * 4 * 4)
    return max(16, min(l, budget_bytes // per_row))


def attention(q: Tensor, k: Tensor, v: Tensor, scale: Optional[float] = None
              ) -> Tensor:
    """softmax(q k^T * scale) v, fp32 softmax; einsum form so forward-mode
    and reverse-mode AD both work on every backend."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    s = torch.einsum("blhd,bshd->bhls", q.float(), k.float()) * scale
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhls,bshd->blhd", p, v.float()).to(v.dtype)


def attention_lse(q: Tensor, k: Tensor, scale: Optional[float] = None) -> Tensor:
    """Natural-log LSE of the scaled scores: (b, H, l)."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    s = torch.einsum("blhd,bshd->bhls", q.float(), k.float()) * scale
    return torch.logsumexp(s, dim=-1)


@torch.no_grad()
def attention_jvp(q: Tensor, k: Tensor, v: Tensor, dq: Tensor, dk: Tensor,
                  dv: Tensor, scale: Optional[float] = None,
                  chunk: Optional[int] = None) -> Tuple[Tensor, Tensor]:
    """(o, do) with
        ds = (dq k^T + q dk^T) scale,  dp = p (ds - rowsum(p ds)),
        do = dp v + p dv.
    Chunked over query rows so the (l, s) score matrix never exceeds ~1 GB."""
    b, l, H, _ = q.shape
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    kf, vf, dkf, dvf = k.float(), v.float(), dk.float(), dv.float()
    step = chunk or _q_chunk(l, k.shape[1], b * H)
    o = torch.empty(b, l, H, v.shape[-1], dtype=v.dtype, device=v.device)
    do = torch.empty_like(o)
    for i in range(0, l, step):
        qf, dqf = q[:, i:i + step].float(), dq[:, i:i + step].float()
        s = torch.einsum("blhd,bshd->bhls", qf, kf) * scale
        ds = (torch.einsum("blhd,bshd->bhls", dqf, kf)
              + torch.einsum("blhd,bshd->bhls", qf, dkf)) * scale
        p = torch.softmax(s, dim=-1)
        dp = p * (ds - (p * ds).sum(-1, keepdim=True))
        o[:, i:i + step] = torch.einsum("bhls,bshd->blhd", p, vf).to(o.dtype)
        do[:, i:i + step] = (torch.einsum("bhls,bshd->blhd", dp, vf)
                             + torch.einsum("bhls,bshd->blhd", p, dvf)).to(o.dtype)
    return o, do


# --------------------------------------------------------------------------
# Attention residual (Kimi-style per-token softmax over residual history)
# --------------------------------------------------------------------------
def attn_res(cands: Sequence[Tensor], w: Tensor, eps: float) -> Tensor:
    """cands: J tensors (..., d), the LAST one is the current prefix sum.
    w: (d,) fused score direction (norm gain * projection weight)."""
    v = torch.stack([c.float() for c in cands], dim=-2)          # (..., J, d)
    r = torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    s = ((v * r) * w.float()).sum(-1)                             # (..., J)
    p = torch.softmax(s, dim=-1)
    return (p.unsqueeze(-1) * v).sum(-2).to(cands[-1].dtype)


@torch.no_grad()
def attn_res_jvp(cands: Sequence[Tensor], dcands: Sequence[Tensor], w: Tensor,
                 eps: float) -> Tuple[Tensor, Tensor]:
    v = torch.stack([c.float() for c in cands], dim=-2)
    dv = torch.stack([c.float() for c in dcands], dim=-2)
    d = v.shape[-1]
    wf = w.float()
    r = torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)       # (..., J, 1)
    vw = (v * wf).sum(-1, keepdim=True)
    dvw = (dv * wf).sum(-1, keepdim=True)
    vdv = (v * dv).sum(-1, keepdim=True) / d
    s = (r * vw).squeeze(-1)
    ds = (r * dvw - r.pow(3) * vw * vdv).squeeze(-1)
    p = torch.softmax(s, dim=-1)
    dp = p * (ds - (p * ds).sum(-1, keepdim=True))
    out = (p.unsqueeze(-1) * v).sum(-2)
    dout = (dp.unsqueeze(-1) * v).sum(-2) + (p.unsqueeze(-1) * dv).sum(-2)
    return out.to(cands[-1].dtype), dout.to(dcands[-1].dtype)


# --------------------------------------------------------------------------
# Newton-Schulz (used by the optimizer tests as the oracle of the kernel)
# --------------------------------------------------------------------------
def newton_schulz(G: Tensor, coeffs: Tuple[float, float, float], steps: int = 5,
                  eps: float = 1e-7, dtype: Optional[torch.dtype] = None) -> Tensor:
    a, b, c = coeffs
    X = G.to(dtype or torch.float32)
    X = X / (X.norm() + eps)
    tr = G.shape[0] > G.shape[1]
    if tr:
        X = X.T
    for _ in range(steps):
        A = X @ X.T
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    return X.T if tr else X
