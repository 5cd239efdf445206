"""Dual-number op layer: every model op takes and returns ``Dual(p, t)``.

``p`` is the primal and takes part in autograd as usual.  ``t`` is the
forward-mode tangent (or ``None``); it is always detached, because the iMF
loss uses du/dt only under stop-gradient (reference ``imf_video.py:533``).
One pass over the network therefore yields u (with its backward graph),
du/dt (no graph) and v, where the reference needs a forward, a checkpoint
recompute and a separate primal+tangent pass (reference
``imf_video.py:495-523``, ``models/mla_jvp_fast.py:310-394``).

Dispatch: CUDA tensors go to the sm_100a kernels in ``ops/cuda.py``; CPU
tensors (and ops without a kernel yet) use the formulas in
``ops/reference.py``.  On a GPU box a missing extension raises instead of
silently falling back (see ``ops/cuda.require``).
"""

from __future__ import annotations

from typing import List, NamedTuple, Optional, Sequence

import torch
import torch.nn.functional as F

from . import reference as ref

Tensor = torch.Tensor


class Dual(NamedTuple):
    p: Tensor
    t: Optional[Tensor] = None

    @property
    def has_t(self) -> bool:
        return self.t is not None

    def map(self, fn) -> "Dual":
        """Apply a LINEAR, parameter-free map to both parts."""
        return Dual(fn(self.p), None if self.t is None else fn(self.t))


def lift(x) -> Dual:
    return x if isinstance(x, Dual) else Dual(x, None)


def _cuda_ops(x: Tensor):
    if x.is_cuda:
        from . import cuda

        return cuda if cuda.available() else None
    return None


# ---------------------------------------------------------------- linear ---
def linear(x: Dual, weight: Tensor, bias: Optional[Tensor] = None) -> Dual:
    """y = x W^T + b ; dy = dx W^T.  On CUDA the primal and tangent rows are
    stacked into ONE GEMM launch (M = 2 b l rows)."""
    w = weight.to(x.p.dtype) if weight.dtype != x.p.dtype else weight
    b = None if bias is None else bias.to(x.p.dtype)
    cu = _cuda_ops(x.p)
    if cu is not None and cu.has("gemm") and x.p.dtype == torch.bfloat16:
        return cu.linear_dual(x, w, b)
    p = F.linear(x.p, w, b)
    t = None
    if x.t is not None:
        with torch.no_grad():
            t = F.linear(x.t, w.detach())
    return Dual(p, t)


# --------------------------------------------------------------- rmsnorm ---
def rmsnorm(x: Dual, weight: Optional[Tensor], eps: float,
            out_dtype: Optional[torch.dtype] = None) -> Dual:
    cu = _cuda_ops(x.p)
    if cu is not None and cu.has("rmsnorm"):
        return cu.rmsnorm_dual(x, weight, eps, out_dtype)
    p = ref.rmsnorm(x.p, weight, eps)
    t = None
    if x.t is not None:
        with torch.no_grad():
            _, t = ref.rmsnorm_jvp(x.p.detach(), x.t,
                                   None if weight is None else weight.detach(), eps)
    od = out_dtype or x.p.dtype       # the fp32 gain must not promote a bf16 stream
    p = p.to(od)
    t = None if t is None else t.to(od)
    return Dual(p, t)


# ------------------------------------------------------------ activation ---
def situ_mul(gate: Dual, up: Dual, beta: float, linear_beta: Optional[float]) -> Dual:
    cu = _cuda_ops(gate.p)
    if cu is not None and cu.has("situ"):
        return cu.situ_dual(gate, up, beta, linear_beta)
    p = ref.situ_mul(gate.p, up.p, beta, linear_beta)
    t = None
    if gate.t is not None:
        with torch.no_grad():
            _, t = ref.situ_mul_jvp(gate.p.detach(), up.p.detach(), gate.t, up.t,
                                    beta, linear_beta)
    return Dual(p, t)


def sigmoid_gate(a: Dual, z: Dual) -> Dual:
    """a * sigmoid(z);  d = da s + a s (1 - s) dz."""
    s = torch.sigmoid(z.p.float())
    p = (a.p.float() * s).to(a.p.dtype)
    t = None
    if a.t is not None:
        with torch.no_grad():
            sd = s.detach()
            t = (a.t.float() * sd
                 + a.p.detach().float() * sd * (1 - sd) * z.t.float()).to(a.t.dtype)
    return Dual(p, t)


def scale_add(res: Optional[Dual], y: Dual, gate: Tensor) -> Dual:
    """res + y * gate (per-channel learned gate, no tangent on the gate).
    Result takes the dtype of ``res`` (the fp32 residual stream) if given."""
    od = y.p.dtype if res is None else res.p.dtype
    p = y.p.to(od) * gate.to(od)
    if res is not None:
        p = res.p + p
    t = None
    if y.t is not None:
        with torch.no_grad():
            t = y.t.to(od) * gate.detach().to(od)
            if res is not None and res.t is not None:
                t = res.t + t
    elif res is not None and res.t is not None:
        t = res.t
    return Dual(p, t)


def add(a: Dual, b: Dual) -> Dual:
    t = None
    if a.t is not None or b.t is not None:
        t = a.t if b.t is None else (b.t if a.t is None else a.t + b.t)
    return Dual(a.p + b.p, t)


# ------------------------------------------------------------------ rope ---
def rope(x: Dual, cos: Tensor, sin: Tensor) -> Dual:
    return x.map(lambda z: ref.rope(z, cos, sin))


# -------------------------------------------------------------- attn_res ---
def attn_res(prefix: Dual, snaps: Sequence[Dual], gain: Tensor, proj_w: Tensor,
             eps: float) -> Dual:
    """Per-token softmax re-mix over [snapshots..., prefix]; reference
    ``models/imf_dit_video.py:287-320``."""
    w = gain.float() * proj_w.reshape(-1).float()
    cands = [s.p for s in snaps] + [prefix.p]
    cu = _cuda_ops(prefix.p)
    if cu is not None and cu.has("attn_res"):
        return cu.attn_res_dual(prefix, list(snaps), w, eps)
    p = ref.attn_res(cands, w, eps)
    t = None
    if prefix.t is not None:
        with torch.no_grad():
            dc = [s.t if s.t is not None else torch.zeros_like(s.p) for s in snaps]
            _, t = ref.attn_res_jvp([c.detach() for c in cands], dc + [prefix.t],
                                    w.detach(), eps)
    return Dual(p, t)


# ------------------------------------------------------------- attention ---
def dense_attention(q: Dual, k: Dual, v: Dual, impl: str = "auto") -> Dual:
    """Dense softmax attention on (b, l, H, d) tensors; scale 1/sqrt(dk).

    impl: "auto" (CUDA kernel on GPU, math on CPU), "math" (einsum formulas,
    forward- and reverse-mode AD capable), "sdpa" (torch fused SDPA primal;
    tangent by the chunked formulas)."""
    cu = _cuda_ops(q.p)
    if impl == "auto" and cu is not None and cu.has("attention"):
        return cu.attention_dual(q, k, v)
    if impl == "sdpa" or (impl == "auto" and q.p.is_cuda):
        qq, kk, vv = (z.transpose(1, 2) for z in (q.p, k.p, v.p))
        if qq.dtype == torch.float32 and qq.is_cuda:
            qq, kk, vv = (z.to(torch.bfloat16) for z in (qq, kk, vv))
        p = F.scaled_dot_product_attention(qq, kk, vv).transpose(1, 2).to(v.p.dtype)
    else:
        p = ref.attention(q.p, k.p, v.p)
    t = None
    if q.t is not None:
        _, t = ref.attention_jvp(q.p.detach(), k.p.detach(), v.p.detach(),
                                 q.t, k.t, v.t)
    return Dual(p, t)


def cat(parts: List[Dual], dim: int) -> Dual:
    p = torch.cat([x.p for x in parts], dim=dim)
    if all(x.t is None for x in parts):
        return Dual(p, None)
    t = torch.cat([x.t if x.t is not None else torch.zeros_like(x.p) for x in parts],
                  dim=dim)
    return Dual(p, t)
