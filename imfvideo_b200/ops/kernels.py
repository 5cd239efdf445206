"""Python bindings (ctypes) and autograd wrappers for ``libimf_b200.so``.

Importing this module registers the available kernels with ``ops.cuda`` so
``ops.dual`` routes CUDA tensors to them.  Launchers return an error code for
bad arguments (raised here as ``ValueError``); kernels report a timed-out
bounded wait through a per-device status word (``check_status``).
"""

from __future__ import annotations

import ctypes
import os
import math
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import cuda as _cuda
from . import reference as ref
from .dual import Dual

_lib = _cuda.require()
c_void_p, c_int, c_int64, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

STATUS_NAMES = {0: "ok", 1: "timeout waiting for a TMA load", 2: "timeout waiting for tcgen05 MMA",
                3: "timeout waiting for softmax warps", 4: "timeout waiting for a free stage",
                5: "bad argument", 6: "timeout waiting for a peer rank",
                7: "timeout waiting for a turn in the fixed-order dQ accumulation"}
_ERR = {-1: "bad shape/stride/alignment", -2: "tensor-map encode failed",
        -3: "kernel launch failed", -4: "size beyond the supported maximum"}

_status: Dict[int, torch.Tensor] = {}


class _LaunchCounter:
    """Number of kernels of this library launched by this process."""
    count = 0


LAUNCHES = _LaunchCounter


def status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device: Optional[torch.device] = None) -> None:
    """Host read of the status word (synchronises); raises if a kernel gave up
    on a bounded wait.  The CUDA context stays usable."""
    devs = list(_status) if device is None else [device.index or 0]
    for d in devs:
        if d in _status:
            code = int(_status[d][0].item())
            if code != 0:
                _status[d].zero_()
                raise RuntimeError(f"imf_b200 kernel status {code}: "
                                   f"{STATUS_NAMES.get(code, 'unknown')}")


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise ValueError(f"{what}: {_ERR.get(rc, rc)}")


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _has(sym: str) -> bool:
    return hasattr(_lib, sym)


# ------------------------------------------------------------------ GEMM ---
if _has("imf_gemm_bf16"):
    _lib.imf_gemm_bf16.restype = c_int
    _lib.imf_gemm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                   c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_float,
                                   c_int, c_void_p, c_void_p]


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         bias: Optional[torch.Tensor] = None, bias_rows: Optional[int] = None,
         alpha: float = 1.0, accumulate: bool = False) -> torch.Tensor:
    """C[M, N] = alpha * op(A) op(B)^T (+ bias).  K-major operands are
    [rows, K]; MN-major operands are [K, rows].  bf16 in, bf16/fp32 out."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    assert out.stride(1) == 1 and out.shape == (M, N)
    fb = None if bias is None else bias.float().contiguous()
    rc = _lib.imf_gemm_bf16(_ptr(a), _ptr(b), _ptr(out), _ptr(fb), M, N, K, a.stride(0),
                            b.stride(0), out.stride(0), int(a_mn), int(b_mn),
                            int(out.dtype == torch.float32),
                            M if bias_rows is None else bias_rows, float(alpha), int(accumulate),
                            _ptr(status_word(a.device)), _stream())
    _check(rc, "imf_gemm_bf16")
    LAUNCHES.count += 1
    return out


if _has("imf_gemm_bf16_splitk"):
    _lib.imf_gemm_splitk_count.restype = c_int
    _lib.imf_gemm_splitk_count.argtypes = [c_int] * 4
    _lib.imf_gemm_bf16_splitk.restype = c_int
    _lib.imf_gemm_bf16_splitk.argtypes = [c_void_p] * 3 + [c_int] * 3 + [c_int64] * 2 + \
        [c_int] * 3 + [c_void_p, c_void_p]
    _lib.imf_splitk_reduce.restype = c_int
    _lib.imf_splitk_reduce.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_int64, c_float,
                                       c_int, c_void_p]

if _has("imf_gemm_fp8"):
    _lib.imf_gemm_fp8.restype = c_int
    _lib.imf_gemm_fp8.argtypes = [c_void_p] * 4 + [c_int] * 3 + [c_int64] * 3 + [c_int, c_int,
                                                                                c_float, c_void_p,
                                                                                c_void_p, c_void_p]
    _lib.imf_quantize_fp8.restype = c_int
    _lib.imf_quantize_fp8.argtypes = [c_void_p, ctypes.c_long, c_int, c_int64, c_void_p, c_int64,
                                      c_void_p, c_void_p, c_void_p]


def quantize_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-tensor e4m3 quantisation of a bf16 matrix [rows, K]: returns the bytes
    ([rows, K rounded up to 16], pad columns zero) and the de-quantisation scale (1 float
    on the device, amax / 448)."""
    assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.stride(1) == 1
    rows, cols = x.shape
    ldo = (cols + 15) // 16 * 16
    out = torch.empty(rows, ldo, dtype=torch.uint8, device=x.device)
    amax = torch.zeros(1, dtype=torch.int32, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    _check(_lib.imf_quantize_fp8(_ptr(x), rows, cols, x.stride(0), _ptr(out), ldo, _ptr(amax),
                                 _ptr(scale), _stream()), "imf_quantize_fp8")
    LAUNCHES.count += 2
    return out, scale


def gemm_fp8(a8: torch.Tensor, sa: torch.Tensor, b8: torch.Tensor, sb: torch.Tensor, *,
             out_dtype: torch.dtype = torch.bfloat16, bias: Optional[torch.Tensor] = None,
             bias_rows: Optional[int] = None) -> torch.Tensor:
    """C[M, N] = sa * sb * A8 B8^T (+ bias) for e4m3 operands from ``quantize_fp8`` ([rows, K]
    bytes each, same padded K), on the tcgen05 ``kind::f8f6f4`` path (twice the bf16 rate).
    Counterpart of the reference's ``_fp8_mm`` (``models/triton_block_jvp.py:80-86``), which
    like this one serves its reduced-precision block variants, not the training default."""
    assert a8.dtype == torch.uint8 and b8.dtype == torch.uint8 and a8.shape[1] == b8.shape[1]
    M, Kp = a8.shape
    N = b8.shape[0]
    out = torch.empty(M, N, dtype=out_dtype, device=a8.device)
    scales = torch.cat([sa.reshape(1), sb.reshape(1)]).float()
    fb = None if bias is None else bias.float().contiguous()
    _check(_lib.imf_gemm_fp8(_ptr(a8), _ptr(b8), _ptr(out), _ptr(fb), M, N, Kp, a8.stride(0),
                             b8.stride(0), out.stride(0), int(out_dtype == torch.float32),
                             M if bias_rows is None else bias_rows, 1.0, _ptr(scales),
                             _ptr(status_word(a8.device)), _stream()), "imf_gemm_fp8")
    LAUNCHES.count += 1
    return out


def linear_fp8(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
               w_cache: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    """y = x w^T (+ bias) with both operands quantised to e4m3 per tensor (the weight
    quantisation can be passed in as ``w_cache`` to reuse it across calls)."""
    x2 = x.reshape(-1, x.shape[-1]).to(torch.bfloat16)
    a8, sa = quantize_fp8(x2 if x2.is_contiguous() else x2.contiguous())
    b8, sb = w_cache if w_cache is not None else quantize_fp8(w.to(torch.bfloat16).contiguous())
    return gemm_fp8(a8, sa, b8, sb, bias=bias).view(*x.shape[:-1], w.shape[0])


SPLITK_TARGET_TILES = 296      # two CTAs per SM on 148 SMs


def gemm_wgrad(dy: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None,
               accumulate: bool = False) -> torch.Tensor:
    """Weight gradient ``out[n_out, n_in] (+)= dy^T x`` for ``dy`` [rows, n_out] and ``x``
    [rows, n_in] (bf16, row-major views with 16-byte row pitch), fp32 result.

    The contraction runs over the token rows, so the output is small and K is long: the K
    range is cut into slices that run as separate tiles (split-K) and are summed in a
    fixed order, straight into ``out`` -- with ``accumulate`` into a gradient buffer that
    already holds other micro-batches' contributions.  Both operands are consumed as they
    are (MN-major), no transposed copy."""
    assert dy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
    assert dy.dim() == 2 and x.dim() == 2 and dy.stride(1) == 1 and x.stride(1) == 1
    rows, M = dy.shape
    N = x.shape[1]
    assert x.shape[0] == rows
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32, device=dy.device)
        accumulate = False
    assert out.dtype == torch.float32 and out.shape == (M, N) and out.stride(1) == 1
    splits = int(_lib.imf_gemm_splitk_count(M, N, rows, SPLITK_TARGET_TILES))
    st = _ptr(status_word(dy.device))
    if splits < 2:
        _check(_lib.imf_gemm_bf16(_ptr(dy), _ptr(x), _ptr(out), None, M, N, rows, dy.stride(0),
                                  x.stride(0), out.stride(0), 1, 1, 1, 0, 1.0, int(accumulate),
                                  st, _stream()), "imf_gemm_bf16 (weight gradient)")
        LAUNCHES.count += 1
        return out
    part = _scratch_buf(dy.device, splits * M * N * 4, "wgrad")
    _check(_lib.imf_gemm_bf16_splitk(_ptr(dy), _ptr(x), _ptr(part), M, N, rows, dy.stride(0),
                                     x.stride(0), 1, 1, splits, st, _stream()),
           "imf_gemm_bf16_splitk")
    _check(_lib.imf_splitk_reduce(_ptr(part), splits, M, N, _ptr(out), out.stride(0), 1.0,
                                  int(accumulate), _stream()), "imf_splitk_reduce")
    LAUNCHES.count += 2
    return out


# ------------------------------------------------------------- attention ---
if _has("imf_attn_fwd"):
    _lib.imf_attn_fwd.restype = c_int
    _lib.imf_attn_fwd.argtypes = [c_void_p] * 9 + [c_int, c_int, c_int, c_int, c_void_p, c_int64,
                                                   c_int64, c_int64, c_float, c_void_p,
                                                   ctypes.c_long, c_void_p, c_void_p]
    _lib.imf_attn_fwd_scratch_bytes.restype = ctypes.c_long
    _lib.imf_attn_fwd_scratch_bytes.argtypes = [c_int, c_int, c_int, c_int]
    _lib.imf_attn_fwd_scratch_bytes_hd.restype = ctypes.c_long
    _lib.imf_attn_fwd_scratch_bytes_hd.argtypes = [c_int, c_int, c_int, c_int, c_int]

ATTN_HEAD_DIMS = (64, 128)

_scratch: Dict[Tuple[int, str], torch.Tensor] = {}


def _scratch_buf(device: torch.device, nbytes: int, tag: str) -> Optional[torch.Tensor]:
    """Per-device grow-only scratch (split-item partials of the persistent
    attention kernels); reused by every call on the same stream order."""
    if nbytes <= 0:
        return None
    key = (device.index or 0, tag)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def _bls(t: torch.Tensor) -> Tuple[int, int, int]:
    assert t.dim() == 4 and t.stride(3) == 1 and t.dtype == torch.bfloat16
    return t.stride(0), t.stride(1), t.stride(2)


def _tma_ok(t: torch.Tensor) -> torch.Tensor:
    """TMA needs a 16-byte-aligned base and 16-byte-multiple strides."""
    if t.stride(3) != 1 or t.data_ptr() % 16 or any((s * 2) % 16 for s in t.stride()[:3]):
        return t.contiguous()
    return t


def attn_fwd(q, k, v, dq=None, dk=None, dv=None, scale: Optional[float] = None,
             need_lse: bool = True):
    """(o, do | None, lse | None) for (B, L, H, head_dim) bf16 tensors, head_dim 64 or 128."""
    B, L, H, hd = q.shape
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    ts = [_tma_ok(t) for t in (q, k, v)]
    tang = dq is not None
    if tang:
        ts += [_tma_ok(t) for t in (dq, dk, dv)]
    strides = []
    for t in ts:
        strides += list(_bls(t))
    arr = (c_int64 * 18)(*(strides + [0] * (18 - len(strides))))
    o = torch.empty(B, L, H, hd, dtype=torch.bfloat16, device=q.device)
    do = torch.empty_like(o) if tang else None
    lse = torch.empty(B, H, L, dtype=torch.float32, device=q.device) if need_lse else None
    nscr = int(_lib.imf_attn_fwd_scratch_bytes_hd(B, L, H, int(tang), hd))
    scr = _scratch_buf(q.device, nscr, "attn_fwd")
    rc = _lib.imf_attn_fwd(_ptr(ts[0]), _ptr(ts[1]), _ptr(ts[2]),
                           _ptr(ts[3]) if tang else None, _ptr(ts[4]) if tang else None,
                           _ptr(ts[5]) if tang else None, _ptr(o), _ptr(do), _ptr(lse), B, L, H,
                           hd, ctypes.cast(arr, c_void_p), o.stride(0), o.stride(1), o.stride(2),
                           float(scale), _ptr(scr), nscr, _ptr(status_word(q.device)), _stream())
    _check(rc, "imf_attn_fwd")
    LAUNCHES.count += 1
    return o, do, lse


if _has("imf_attn_bwd"):
    _lib.imf_attn_bwd.restype = c_int
    _lib.imf_attn_bwd.argtypes = [c_void_p] * 9 + [c_int] * 4 + [c_void_p] * 4 + \
        [c_float, c_void_p, ctypes.c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
         c_void_p, c_void_p]
    _lib.imf_attn_bwd_scratch_bytes.restype = ctypes.c_long
    _lib.imf_attn_bwd_scratch_bytes.argtypes = [c_int, c_int, c_int]
    _lib.imf_attn_bwd_scratch_bytes_hd.restype = ctypes.c_long
    _lib.imf_attn_bwd_scratch_bytes_hd.argtypes = [c_int, c_int, c_int, c_int]


# True: the dQ tiles of the attention backward are added in a fixed order, which makes a whole
# training step bit-identical from run to run (every other reduction of the library already has
# a fixed order) at 13 % (head_dim 64) to 34 % (head_dim 128) of that kernel's time.  False
# (default; IMF_DETERMINISTIC=1 in the environment or ``run.deterministic`` in the config turn
# it on): the tiles land in arrival order.
DETERMINISTIC = os.environ.get("IMF_DETERMINISTIC", "0") == "1"


def set_deterministic(on: bool) -> None:
    global DETERMINISTIC
    DETERMINISTIC = bool(on)


def attn_bwd(q, k, v, o, lse, go, scale: Optional[float] = None,
             gv_out: Optional[torch.Tensor] = None, qlist: Optional[torch.Tensor] = None,
             qflags: Optional[torch.Tensor] = None, qrank: Optional[torch.Tensor] = None,
             dq_add: Optional[torch.Tensor] = None):
    """(dq, dk, dv) of dense attention; ``gv_out`` lets dv land in a strided
    view (e.g. the value band of the kv up-projection gradient).  With
    ``qlist`` / ``qflags`` (see ``ops.sparse.kv_lists``) the same kernel
    runs the block-sparse backward: each 128-row K/V tile walks only the query
    tiles that attend it; ``qrank`` (same source) gives the entries' places in the fixed
    order of dQ additions (without it the block-sparse dQ adds land in arrival order).
    ``dq_add`` (fp32, (B, L, H, 64) contiguous, head_dim 64): added to dq before it is rounded
    to bf16 (the query gradient of another branch of the same attention module)."""
    B, L, H, hd = q.shape
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    ts = [_tma_ok(t) for t in (q, k, v, go)]
    strides = []
    for t in ts:
        strides += list(_bls(t))
    arr = (c_int64 * 12)(*strides)
    o = o if o.stride(3) == 1 else o.contiguous()
    if dq_add is not None:
        assert dq_add.dtype == torch.float32 and dq_add.shape == (B, L, H, hd) \
            and dq_add.is_contiguous() and hd == 64
    dq = torch.empty(B, L, H, hd, dtype=torch.bfloat16, device=q.device)
    dk = torch.empty(B, L, H, hd, dtype=torch.bfloat16, device=q.device)
    dv = gv_out if gv_out is not None else torch.empty(B, L, H, hd, dtype=torch.bfloat16,
                                                        device=q.device)
    if dv.stride(3) != 1 or dv.data_ptr() % 16 or any(s_ % 8 for s_ in dv.stride()[:3]):
        raise ValueError("dv output needs 16-byte aligned rows")
    i3 = lambda t: (c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    nscr = int(_lib.imf_attn_bwd_scratch_bytes_hd(B, L, H, hd))
    scr = _scratch_buf(q.device, nscr, "attn_bwd")
    rc = _lib.imf_attn_bwd(_ptr(ts[0]), _ptr(ts[1]), _ptr(ts[2]), _ptr(o), _ptr(ts[3]),
                           _ptr(lse), _ptr(dq), _ptr(dk), _ptr(dv), B, L, H, hd,
                           ctypes.cast(arr, c_void_p), ctypes.cast(i3(o), c_void_p),
                           ctypes.cast(i3(dk), c_void_p), ctypes.cast(i3(dv), c_void_p),
                           float(scale), _ptr(scr), nscr, _ptr(qlist), _ptr(qflags), _ptr(qrank),
                           0 if qlist is None else qlist.shape[-1], int(DETERMINISTIC),
                           _ptr(dq_add), _ptr(status_word(q.device)), _stream())
    _check(rc, "imf_attn_bwd")
    LAUNCHES.count += 3
    return dq, dk, dv


# ------------------------------------------------- autograd: attention -----
def _sdpa_backward(q, k, v, go):
    """Temporary reverse-mode fallback (library SDPA recompute) used only when
    the library lacks ``imf_attn_bwd``."""
    with torch.enable_grad():
        qq, kk, vv = (t.detach().transpose(1, 2).requires_grad_(True) for t in (q, k, v))
        oo = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv)
        gq, gk, gv = torch.autograd.grad(oo, (qq, kk, vv), go.transpose(1, 2))
    return gq.transpose(1, 2), gk.transpose(1, 2), gv.transpose(1, 2)


class _AttnFn(torch.autograd.Function):
    """o (and the detached tangent do) from the fused kernel; reverse mode
    through the primal only."""

    @staticmethod
    def forward(ctx, q, k, v, dq, dk, dv):
        need_bwd = any(ctx.needs_input_grad[:3])
        o, do, lse = attn_fwd(q, k, v, dq, dk, dv, need_lse=need_bwd)
        if need_bwd:
            ctx.save_for_backward(q, k, v, o, lse)
        if do is None:
            do = o.new_empty(0)
        ctx.mark_non_differentiable(do)
        return o, do

    @staticmethod
    def backward(ctx, go, _gdo):
        q, k, v, o, lse = ctx.saved_tensors
        if _has("imf_attn_bwd"):
            gq, gk, gv = attn_bwd(q, k, v, o, lse, go.contiguous())
        else:
            gq, gk, gv = _sdpa_backward(q, k, v, go)
        return gq, gk, gv, None, None, None


def attention_dual(q: Dual, k: Dual, v: Dual) -> Dual:
    if q.p.dtype != torch.bfloat16 or q.p.shape[-1] not in ATTN_HEAD_DIMS \
            or v.p.shape[-1] != q.p.shape[-1]:
        raise ValueError("attention kernel needs bf16 tensors with head_dim 64 or 128; got "
                         f"{q.p.dtype}, qk {q.p.shape[-1]}, v {v.p.shape[-1]}")
    if q.t is not None:
        o, do = _AttnFn.apply(q.p, k.p, v.p, q.t, k.t, v.t)
        return Dual(o, do)
    o, _ = _AttnFn.apply(q.p, k.p, v.p, None, None, None)
    return Dual(o, None)


# ---------------------------------------------------- autograd: linear -----
def _stacked(xp: torch.Tensor, xt: Optional[torch.Tensor], kdim: int):
    """2-D [rows, K] view over primal (+ tangent) rows; zero-copy when the
    tangent sits right behind the primal in memory."""
    a = xp.reshape(-1, kdim)
    if xt is None:
        return a, a.shape[0]
    b = xt.reshape(-1, kdim)
    if (a.is_contiguous() and b.is_contiguous()
            and b.data_ptr() == a.data_ptr() + a.numel() * a.element_size()
            and a.untyped_storage().data_ptr() == b.untyped_storage().data_ptr()):
        return torch.as_strided(a, (a.shape[0] * 2, kdim), (kdim, 1)), a.shape[0]
    return torch.cat([a, b], dim=0), a.shape[0]


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xp, xt, w, bias):
        kdim = xp.shape[-1]
        x2, mp = _stacked(xp, xt, kdim)
        if x2.stride(0) % 8 or x2.data_ptr() % 16:
            x2 = x2.contiguous()
        y = gemm(x2, w, bias=bias, bias_rows=mp)
        n = w.shape[0]
        yp = y[:mp].view(*xp.shape[:-1], n)
        yt = y[mp:].view(*xp.shape[:-1], n) if xt is not None else y.new_empty(0)
        ctx.save_for_backward(xp, w)
        ctx.has_bias = bias is not None
        ctx.mark_non_differentiable(yt)
        return yp, yt

    @staticmethod
    def backward(ctx, gyp, _gyt):
        xp, w = ctx.saved_tensors
        g2 = gyp.reshape(-1, gyp.shape[-1])
        x2 = xp.reshape(-1, xp.shape[-1])
        gx = gw = gb = None
        # own GEMM when the operands meet its 16-byte rules (bf16, contiguous rows, widths
        # that are multiples of 8); otherwise the framework's matmul
        ok = (g2.dtype == torch.bfloat16 and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
              and g2.shape[1] % 8 == 0 and x2.shape[1] % 8 == 0)
        if ok:
            g2 = g2 if (g2.is_contiguous() and g2.data_ptr() % 16 == 0) else g2.contiguous()
            x2 = x2 if (x2.is_contiguous() and x2.data_ptr() % 16 == 0) else x2.contiguous()
        if ctx.needs_input_grad[0]:
            gx = (gemm(g2, w, b_mn=True) if ok else g2 @ w).view_as(xp)
        if ctx.needs_input_grad[2]:
            gw = gemm_wgrad(g2, x2).to(w.dtype) if ok else g2.t() @ x2
        if ctx.has_bias and ctx.needs_input_grad[3]:
            gb = g2.float().sum(0).to(g2.dtype)
        return gx, None, gw, gb


def linear_dual(x: Dual, w: torch.Tensor, bias: Optional[torch.Tensor]) -> Dual:
    if x.p.shape[-1] % 8:
        raise ValueError(f"GEMM K={x.p.shape[-1]} must be a multiple of 8 (pad the operand)")
    w = w if w.is_contiguous() else w.contiguous()
    yp, yt = _LinearFn.apply(x.p, x.t, w, bias)
    return Dual(yp, yt if x.t is not None else None)


if _has("imf_gemm_bf16"):
    _cuda.register("gemm", linear_dual=linear_dual)
if _has("imf_attn_fwd"):
    _cuda.register("attention", attention_dual=attention_dual)
if _has("imf_resnorm") and _has("imf_gemm_bf16") and _has("imf_attn_fwd"):
    _cuda.register("block")


# ------------------------------------------------ batched GEMM / Newton-Schulz
if _has("imf_gemm_bf16_batched"):
    _lib.imf_gemm_bf16_batched.restype = c_int
    _lib.imf_gemm_bf16_batched.argtypes = [c_void_p] * 4 + [c_int] * 3 + [c_int64] * 3 + [c_int] + \
        [c_int64] * 3 + [c_int] * 3 + [c_float, c_float, c_void_p, c_void_p]


_HAS_SYM = _has("imf_gemm_bf16_batched_sym")
if _HAS_SYM:
    _lib.imf_gemm_bf16_batched_sym.restype = c_int
    _lib.imf_gemm_bf16_batched_sym.argtypes = [c_void_p] * 4 + [c_int] * 2 + [c_int64] * 3 + \
        [c_int] + [c_int64] * 3 + [c_int, c_float, c_float, c_void_p, c_void_p]


def gemm_batched(a, b, *, a_mn=False, b_mn=False, cin=None, alpha=1.0, beta=0.0, out=None,
                 out_dtype=torch.bfloat16, sym=False):
    """out[z] = alpha * op(a[z]) op(b[z])^T + beta * cin[z] for 3-D bf16 tensors.
    ``sym``: the caller knows the result (and ``cin``) to be symmetric -- X X^T, X^T X, or
    A A with A symmetric: only the tiles on and above the diagonal are computed and the
    epilogue writes their mirror images (bf16 output, both operands of the same major)."""
    assert a.dim() == 3 and b.dim() == 3 and a.stride(2) == 1 and b.stride(2) == 1
    Z = a.shape[0]
    M, K = (a.shape[2], a.shape[1]) if a_mn else (a.shape[1], a.shape[2])
    N, Kb = (b.shape[2], b.shape[1]) if b_mn else (b.shape[1], b.shape[2])
    assert K == Kb and b.shape[0] == Z
    if out is None:
        out = torch.empty(Z, M, N, dtype=out_dtype, device=a.device)
    assert out.stride(2) == 1 and (cin is None or (cin.shape == out.shape and
                                                   cin.stride() == out.stride()
                                                   and cin.dtype == out.dtype))
    if (sym and _HAS_SYM and M == N and a_mn == b_mn and out.dtype == torch.bfloat16
            and out.stride(1) % 8 == 0 and out.data_ptr() % 16 == 0
            and (Z == 1 or out.stride(0) % 8 == 0)):
        rc = _lib.imf_gemm_bf16_batched_sym(_ptr(a), _ptr(b), _ptr(out), _ptr(cin), M, K,
                                            a.stride(1), b.stride(1), out.stride(1), Z, a.stride(0),
                                            b.stride(0), out.stride(0), int(a_mn), float(alpha),
                                            float(beta), _ptr(status_word(a.device)), _stream())
        _check(rc, "imf_gemm_bf16_batched_sym")
        LAUNCHES.count += 1
        return out
    rc = _lib.imf_gemm_bf16_batched(_ptr(a), _ptr(b), _ptr(out), _ptr(cin), M, N, K, a.stride(1),
                                    b.stride(1), out.stride(1), Z, a.stride(0), b.stride(0),
                                    out.stride(0), int(a_mn), int(b_mn),
                                    int(out.dtype == torch.float32), float(alpha), float(beta),
                                    _ptr(status_word(a.device)), _stream())
    _check(rc, "imf_gemm_bf16_batched")
    LAUNCHES.count += 1
    return out


if _has("imf_ns_prepare"):
    _lib.imf_ns_prepare.restype = c_int
    _lib.imf_ns_prepare.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                    c_float, c_void_p]

_ns_ws: Dict[Tuple[int, int, int, int], Tuple[torch.Tensor, ...]] = {}


def _ns_workspace(dev: torch.device, k: int, n: int, mp: int, g: int):
    """X, Y (k, n, mp), A, B (k, g, g) bf16 and the norm partials, allocated once per shape
    batch and reused by every later step (the optimizer calls with the same shapes)."""
    key = (dev.index or 0, k, n, mp)
    ws = _ns_ws.get(key)
    if ws is None:
        bf = dict(dtype=torch.bfloat16, device=dev)
        ws = (torch.zeros(k, n, mp, **bf), torch.zeros(k, n, mp, **bf),
              torch.empty(k, g, g, **bf), torch.empty(k, g, g, **bf),
              torch.empty(k * 32, dtype=torch.float64, device=dev))
        _ns_ws[key] = ws
    return ws


def newton_schulz(G: torch.Tensor, coeffs, steps: int = 5, eps: float = 1e-7,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Quintic Newton-Schulz on a batch (k, n, m) with the tcgen05 GEMM:
    per iteration A = X X^T (or X^T X when n > m), B = b A + c A A (both symmetric: only the
    tiles on and above the diagonal are computed, the epilogue mirrors them),
    X <- a X + B X (or X B), three launches for the whole batch.  The Gram
    side is chosen by operand major flags, so no transposed copy is made.
    Normalisation, cast and padding are one two-launch kernel; the iterates live in
    a workspace kept between calls; with ``out`` (bf16 (k, n, m), m a multiple of 8)
    the last iteration writes the result there."""
    a_, b_, c_ = coeffs
    k, n, m = G.shape
    if min(n, m) < 8 or (n > m and m % 8):
        return None                 # tiny / odd Gram side: the caller uses the torch path
    mp = (m + 7) // 8 * 8
    small_rows = n <= m
    g = n if small_rows else mp
    X, Y, A, B, part = _ns_workspace(G.device, k, n, mp, g)
    Gf = G if (G.dtype == torch.float32 and G.is_contiguous()) else G.float().contiguous()
    if _has("imf_ns_prepare"):
        _check(_lib.imf_ns_prepare(_ptr(Gf), _ptr(X), k, n, m, mp, _ptr(part), float(eps),
                                   _stream()), "imf_ns_prepare")
        LAUNCHES.count += 2
    else:
        nrm = Gf.flatten(1).norm(dim=1).view(k, 1, 1) + eps
        X.zero_()
        X[:, :, :m] = (Gf / nrm).to(torch.bfloat16)
    if mp != m:
        Y.zero_()        # the pad columns of the other iterate stay zero through a X + B X
    direct = (out is not None and mp == m and out.dtype == torch.bfloat16 and out.is_contiguous()
              and out.shape == (k, n, m))
    # upper tiles + mirror pays from four tiles along the Gram side on (measured: 24 x 1024 x
    # 1024 1.10 -> 0.93 ms, 30 x 1536 x 1536 3.93 -> 2.93 ms, but 64 x 256 x 256 0.25 -> 0.28 ms)
    sym = g >= 512 and os.environ.get("IMF_NS_SYM", "1") != "0"     # IMF_NS_SYM=0: full products
    for it in range(steps):
        dst = out if (direct and it == steps - 1) else Y
        if small_rows:
            gemm_batched(X, X, out=A, sym=sym)                               # X X^T
            gemm_batched(A, A, cin=A, alpha=c_, beta=b_, out=B, sym=sym)     # b A + c A A
            gemm_batched(B, X, b_mn=True, cin=X, alpha=1.0, beta=a_, out=dst)  # a X + B X
        else:
            gemm_batched(X, X, a_mn=True, b_mn=True, out=A, sym=sym)         # X^T X
            gemm_batched(A, A, cin=A, alpha=c_, beta=b_, out=B, sym=sym)
            gemm_batched(X, B, cin=X, alpha=1.0, beta=a_, out=dst)           # a X + X B
        X, Y = dst, X
    if direct:
        return out
    res = X[:, :, :m]
    if out is not None:
        out.copy_(res)
        return out
    return res.clone()      # the workspace is reused by the next call


if _has("imf_gemm_bf16_batched"):
    _cuda.register("newton_schulz", newton_schulz=newton_schulz)
