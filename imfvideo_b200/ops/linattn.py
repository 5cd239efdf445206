"""Linear-attention complement branch of SLA2 / cube attention on this
library's kernels (``csrc/linattn.cu`` + the tcgen05 GEMM for the mask
product): forward with optional tangent, and reverse mode.

Tensors are ``(B, L, H, 64)`` bf16 in the model's layout (any batch / row / head
strides, last dim contiguous).  ``sel`` is the ``(B, H, Mb, T)`` list of key
blocks each query block attends in the softmax branch; the linear branch
covers the remaining key blocks below ``n_comp`` (reference
models/sla2_vendor/core.py SLA2 forward, models/triton_sla2_jvp.py
``_linear_jvp``).
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import kernels as K

_lib = K._lib
vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_long

AVAILABLE = K._has("imf_lin_states")
if AVAILABLE:
    _lib.imf_lin_state_elems.restype = ci
    LSTATE = int(_lib.imf_lin_state_elems())
    _lib.imf_lin_states.restype = ci
    _lib.imf_lin_states.argtypes = [vp] * 7 + [ci] * 8 + [vp, vp]
    _lib.imf_lin_apply.restype = ci
    _lib.imf_lin_apply.argtypes = [vp] * 9 + [ci] * 5 + [vp, vp]
    _lib.imf_lin_bwd_rows.restype = ci
    _lib.imf_lin_bwd_rows.argtypes = [vp] * 10 + [ci] * 5 + [vp, vp]
    _lib.imf_lin_bwd_kv.restype = ci
    _lib.imf_lin_bwd_kv.argtypes = [vp] * 7 + [ci] * 5 + [vp, vp]
    if K._has("imf_comp_mask"):
        _lib.imf_comp_mask.restype = ci
        _lib.imf_comp_mask.argtypes = [vp, vp] + [ci] * 5 + [vp]
else:
    LSTATE = 64 * 68


def _strides(*ts) -> "ctypes.Array":
    flat = []
    for t in ts:
        if t is None:
            flat += [0, 0, 0]
        else:
            assert t.dim() == 4 and t.stride(3) == 1, (t.shape, t.stride())
            flat += [t.stride(0), t.stride(1), t.stride(2)]
    return (ctypes.c_int64 * len(flat))(*flat)


def _pad4(n: int) -> int:
    return (n + 3) // 4 * 4


def comp_mask(sel: torch.Tensor, Mb: int, Nb: int, transpose: bool = False) -> torch.Tensor:
    """0/1 complement of the selection, duplicated for the (hi, lo) halves of the states:
    ``(B*H, Mb, 2*pad4(Nb))`` bf16, or the transposed ``(B*H, Nb, 2*pad4(Mb))``."""
    B, H = sel.shape[:2]
    if AVAILABLE and sel.is_cuda and sel.dtype == torch.int32 and K._has("imf_comp_mask"):
        sel = sel.contiguous()
        rows, cols = (Nb, Mb) if transpose else (Mb, Nb)
        out = torch.empty(B * H, rows, 2 * _pad4(cols), dtype=torch.bfloat16, device=sel.device)
        rc = _lib.imf_comp_mask(K._ptr(sel), K._ptr(out), B * H, Mb, Nb, sel.shape[-1],
                                int(transpose), K._stream())
        K._check(rc, "imf_comp_mask")
        K.LAUNCHES.count += 2 if transpose else 1
        return out
    cm = torch.ones(B, H, Mb, Nb, dtype=torch.bfloat16, device=sel.device)
    cm.scatter_(-1, sel.long(), 0.0)
    if transpose:
        cm = cm.transpose(-1, -2)
        rows, cols = Nb, Mb
    else:
        rows, cols = Mb, Nb
    cp = _pad4(cols)
    out = torch.zeros(B * H, rows, 2 * cp, dtype=torch.bfloat16, device=sel.device)
    cmv = cm.reshape(B * H, rows, cols)
    out[:, :, :cols] = cmv
    out[:, :, cp:cp + cols] = cmv
    return out


def states(x, dx, y, dy, w, bs: int, lim: int) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Per block of ``bs`` rows: [softmax(x)^T y | softmax(x)^T w] (and the tangent) as bf16
    (hi, lo) rows: ``(B*H, 2*pad4(nblk), LSTATE)``."""
    B, L, H, D = x.shape
    assert D == 64 and x.dtype == torch.bfloat16
    nblk = -(-L // bs)
    nbp = _pad4(nblk)
    mk = torch.zeros if nbp != nblk else torch.empty
    out = mk(B * H, 2 * nbp, LSTATE, dtype=torch.bfloat16, device=x.device)
    dout = mk(B * H, 2 * nbp, LSTATE, dtype=torch.bfloat16, device=x.device) if dx is not None else None
    y_fp32 = y.dtype == torch.float32
    assert y_fp32 or y.dtype == torch.bfloat16
    if w is not None:
        assert w.dtype == torch.float32 and w.is_contiguous() and w.shape == (B, H, L)
    rc = _lib.imf_lin_states(K._ptr(x), K._ptr(dx), K._ptr(y), K._ptr(dy), K._ptr(w), K._ptr(out),
                             K._ptr(dout), B, L, H, bs, nblk, nbp, lim, int(y_fp32),
                             _strides(x, dx, y, dy), K._stream())
    K._check(rc, "imf_lin_states")
    K.LAUNCHES.count += 1
    return out, dout


def forward(q, k, v, dq, dk, dv, o_s, do_s, sel, a_rows, qblk: int, bk: int,
            n_comp: Optional[int]):
    """o = a o_s + (1 - a) o_l (and its tangent).  Returns (o, do, C) with C the
    ``(B*H, Mb, LSTATE)`` fp32 complement states (kept for reverse mode)."""
    B, L, H, D = q.shape
    Mb, Nb = -(-L // qblk), -(-L // bk)
    lim = L if n_comp is None else min(L, n_comp * bk)
    tangent = dq is not None
    S2, dS2 = states(k, dk if tangent else None, v, dv if tangent else None, None, bk, lim)
    cm2 = comp_mask(sel, Mb, Nb)
    C = K.gemm_batched(cm2, S2, b_mn=True, out_dtype=torch.float32)
    dC = K.gemm_batched(cm2, dS2, b_mn=True, out_dtype=torch.float32) if tangent else None
    a_rows = a_rows.detach().float().contiguous()
    o = torch.empty(B, L, H, D, dtype=torch.bfloat16, device=q.device)
    do = torch.empty_like(o) if tangent else None
    rc = _lib.imf_lin_apply(K._ptr(q), K._ptr(dq), K._ptr(o_s), K._ptr(do_s), K._ptr(C),
                            K._ptr(dC), K._ptr(a_rows), K._ptr(o), K._ptr(do), B, L, H, Mb, qblk,
                            _strides(q, dq, o_s, do_s, o, do), K._stream())
    K._check(rc, "imf_lin_apply")
    K.LAUNCHES.count += 1
    return o, do, C


def backward_rows(q, o_s, go, C, a_rows, qblk: int):
    """Row side of reverse mode.  Returns (gq_l fp32, gnum fp32, gden, ga_row, g_os bf16)."""
    B, L, H, D = q.shape
    Mb = -(-L // qblk)
    dev = q.device
    gq = torch.empty(B, L, H, D, dtype=torch.float32, device=dev)
    gnum = torch.empty(B, L, H, D, dtype=torch.float32, device=dev)
    gden = torch.empty(B, H, L, dtype=torch.float32, device=dev)
    ga_row = torch.empty(B, H, L, dtype=torch.float32, device=dev)
    g_os = torch.empty(B, L, H, D, dtype=torch.bfloat16, device=dev)
    a_rows = a_rows.detach().float().contiguous()
    rc = _lib.imf_lin_bwd_rows(K._ptr(q), K._ptr(o_s), K._ptr(go), K._ptr(C), K._ptr(a_rows),
                               K._ptr(gq), K._ptr(gnum), K._ptr(gden), K._ptr(ga_row),
                               K._ptr(g_os), B, L, H, Mb, qblk, _strides(q, o_s, go, g_os),
                               K._stream())
    K._check(rc, "imf_lin_bwd_rows")
    K.LAUNCHES.count += 1
    return gq, gnum, gden, ga_row, g_os


def backward_kv(q, k, v, gnum, gden, sel, gk_s, gv_s, qblk: int, bk: int, n_comp: Optional[int],
                gv_out: Optional[torch.Tensor] = None):
    """Key side of reverse mode: dL/dC from (phi(q), gnum | gden), the transposed mask
    product, then dK / dV of the linear branch added to the sparse branch's (gk_s, gv_s)."""
    B, L, H, D = q.shape
    Mb, Nb = -(-L // qblk), -(-L // bk)
    lim = L if n_comp is None else min(L, n_comp * bk)
    gC2, _ = states(q, None, gnum, None, gden, qblk, L)
    cmT2 = comp_mask(sel, Mb, Nb, transpose=True)
    gS = K.gemm_batched(cmT2, gC2, b_mn=True, out_dtype=torch.float32)       # (B*H, Nb, LSTATE)
    gk = torch.empty(B, L, H, D, dtype=torch.bfloat16, device=q.device)
    gv = gv_out if gv_out is not None else torch.empty_like(gk)
    rc = _lib.imf_lin_bwd_kv(K._ptr(k), K._ptr(v), K._ptr(gk_s), K._ptr(gv_s), K._ptr(gS),
                             K._ptr(gk), K._ptr(gv), B, L, H, Nb, lim,
                             _strides(k, v, gk_s, gv_s, gk, gv), K._stream())
    K._check(rc, "imf_lin_bwd_kv")
    K.LAUNCHES.count += 1
    return gk, gv
