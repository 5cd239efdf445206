"""Layout kernels around the transformer (``csrc/patch.cu``): patch rows of a
latent video and back, row permutation of a token sequence, sinusoidal scalar
embedding.  Each function has an autograd rule built from the adjoint kernel
(gather <-> scatter, permutation <-> inverse permutation) and falls back to the
reshape / index formulas for CPU tensors.

Reference: ``VideoPatchEmbedder`` / ``unpatchify`` / ``timestep_embedding`` of
models/imf_dit_video.py and the tile gathers of models/sla2_cube.py.
"""

from __future__ import annotations

import ctypes
import math
from typing import Tuple

import torch

from . import kernels as K

_lib = K._lib
vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

AVAILABLE = K._has("imf_patch_gather")
if AVAILABLE:
    _lib.imf_patch_gather.restype = ci
    _lib.imf_patch_gather.argtypes = [vp, vp] + [ci] * 11 + [vp]
    _lib.imf_patch_scatter.restype = ci
    _lib.imf_patch_scatter.argtypes = [vp, vp] + [ci] * 10 + [vp]
    _lib.imf_permute_rows.restype = ci
    _lib.imf_permute_rows.argtypes = [vp, vp, vp] + [ci] * 4 + [vp]
    _lib.imf_sinusoid.restype = ci
    _lib.imf_sinusoid.argtypes = [vp, vp, vp, ci, ci, cf, vp]

_OK_DTYPES = (torch.float32, torch.bfloat16)


def _on_kernels(t: torch.Tensor) -> bool:
    return (AVAILABLE and t.is_cuda and t.dtype in _OK_DTYPES
            and not torch._C._are_functorch_transforms_active())


# ------------------------------------------------------------------ formulas ---
def gather_formula(x: torch.Tensor, patch, c_last: bool) -> torch.Tensor:
    b, c, t, h, w = x.shape
    pt, ph, pw = patch
    x = x.reshape(b, c, t // pt, pt, h // ph, ph, w // pw, pw)
    x = x.permute(0, 2, 4, 6, 3, 5, 7, 1) if c_last else x.permute(0, 2, 4, 6, 1, 3, 5, 7)
    return x.reshape(b, (t // pt) * (h // ph) * (w // pw), c * pt * ph * pw)


def scatter_formula(rows: torch.Tensor, shape, patch, c_last: bool) -> torch.Tensor:
    b, c, t, h, w = shape
    pt, ph, pw = patch
    gt, gh, gw = t // pt, h // ph, w // pw
    if c_last:
        x = rows.reshape(b, gt, gh, gw, pt, ph, pw, c).permute(0, 7, 1, 4, 2, 5, 3, 6)
    else:
        x = rows.reshape(b, gt, gh, gw, c, pt, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7)
    return x.reshape(b, c, t, h, w)


# ------------------------------------------------------------------- kernels ---
def _gather(x: torch.Tensor, patch, c_last: bool, out_dtype: torch.dtype) -> torch.Tensor:
    x = x.contiguous()
    b, c, t, h, w = x.shape
    pt, ph, pw = patch
    n = (t // pt) * (h // ph) * (w // pw)
    rows = torch.empty(b, n, c * pt * ph * pw, dtype=out_dtype, device=x.device)
    K._check(_lib.imf_patch_gather(K._ptr(x), K._ptr(rows), b, c, t, h, w, pt, ph, pw, int(c_last),
                                   int(x.dtype == torch.bfloat16),
                                   int(out_dtype == torch.bfloat16), K._stream()),
             "imf_patch_gather")
    K.LAUNCHES.count += 1
    return rows


def _scatter(rows: torch.Tensor, shape, patch, c_last: bool) -> torch.Tensor:
    rows = rows.contiguous()
    b, c, t, h, w = shape
    pt, ph, pw = patch
    x = torch.empty(b, c, t, h, w, dtype=torch.float32, device=rows.device)
    K._check(_lib.imf_patch_scatter(K._ptr(rows), K._ptr(x), b, c, t, h, w, pt, ph, pw,
                                    int(c_last), int(rows.dtype == torch.bfloat16), K._stream()),
             "imf_patch_scatter")
    K.LAUNCHES.count += 1
    return x


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, patch, c_last):
        ctx.shape, ctx.patch, ctx.c_last, ctx.dtype = tuple(x.shape), patch, c_last, x.dtype
        return _gather(x, patch, c_last, x.dtype)

    @staticmethod
    def backward(ctx, g):
        return _scatter(g, ctx.shape, ctx.patch, ctx.c_last).to(ctx.dtype), None, None


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, shape, patch, c_last):
        ctx.patch, ctx.c_last, ctx.dtype = patch, c_last, rows.dtype
        return _scatter(rows, shape, patch, c_last)

    @staticmethod
    def backward(ctx, g):
        return _gather(g, ctx.patch, ctx.c_last, ctx.dtype), None, None, None


def patch_rows(x: torch.Tensor, patch, c_last: bool = False) -> torch.Tensor:
    """(B, C, T, H, W) -> (B, N, C*pt*ph*pw) patch rows, same dtype."""
    patch = tuple(int(p) for p in patch)
    if not _on_kernels(x):
        return gather_formula(x, patch, c_last)
    return _Gather.apply(x, patch, c_last)


def unpatch_rows(rows: torch.Tensor, shape, patch, c_last: bool = True) -> torch.Tensor:
    """(B, N, F) patch rows (bf16 or fp32) -> (B, C, T, H, W) fp32."""
    patch = tuple(int(p) for p in patch)
    if not _on_kernels(rows):
        return scatter_formula(rows.float(), shape, patch, c_last)
    return _Scatter.apply(rows, tuple(int(s) for s in shape), patch, c_last)


def _permute(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    src = src.contiguous()
    B, L, D = src.shape
    dst = torch.empty(B, idx.numel(), D, dtype=src.dtype, device=src.device)
    K._check(_lib.imf_permute_rows(K._ptr(src), K._ptr(dst), K._ptr(idx), B, L, idx.numel(),
                                   D * src.element_size(), K._stream()), "imf_permute_rows")
    K.LAUNCHES.count += 1
    return dst


class _Permute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src, idx, inv):
        ctx.save_for_backward(inv, idx)
        return _permute(src, idx)

    @staticmethod
    def backward(ctx, g):
        inv, idx = ctx.saved_tensors
        return _permute(g, inv), None, None


def permute_rows(z: torch.Tensor, idx: torch.Tensor, inv: torch.Tensor) -> torch.Tensor:
    """``z[:, idx]`` for a permutation ``idx`` of the rows of ``z`` (B, L, D) with inverse
    ``inv`` (the backward is the same kernel with ``inv``)."""
    ok = (_on_kernels(z) and z.dim() == 3 and idx.dtype == torch.int64 and idx.is_cuda
          and idx.numel() == z.shape[1] == inv.numel()
          and (z.shape[2] * z.element_size()) % 16 == 0)
    if not ok:
        return z[:, idx]
    return _Permute.apply(z, idx.contiguous(), inv.contiguous())


def sinusoid(t: torch.Tensor, dim: int, max_period: float = 10000.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos|sin features of a scalar per batch element and their derivative w.r.t. it:
    two (B, dim) fp32 tensors in one launch (no autograd: the scalar is an input)."""
    assert AVAILABLE and t.is_cuda and t.dim() == 1
    t = t.detach().float().contiguous()
    emb = torch.empty(t.shape[0], dim, dtype=torch.float32, device=t.device)
    demb = torch.empty_like(emb)
    K._check(_lib.imf_sinusoid(K._ptr(t), K._ptr(emb), K._ptr(demb), t.shape[0], dim,
                               float(max_period), K._stream()), "imf_sinusoid")
    K.LAUNCHES.count += 1
    return emb, demb
