"""Python bindings (ctypes) and autograd wrappers for ``libimf_b200.so``.

Importing this module registers the available kernels with ``ops.cuda`` so
``ops.dual`` routes CUDA tensors to them.  Launchers return an error code for
bad arguments (raised here as ``ValueError``); kernels report a timed-out
bounded wait through a per-device status word (``check_status``).
"""

from __future__ import annotations

import ctypes
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
                5: "bad argument", 6: "timeout waiting for a peer rank"}
_ERR = {-1: "bad shape/stride/alignment", -2: "tensor-map encode failed",
        -3: "kernel launch failed", -4: "size beyond the supported maximum"}

_status: Dict[int, torch.Tensor] = {}


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
    return out


# ------------------------------------------------------------- attention ---
if _has("imf_attn_fwd"):
    _lib.imf_attn_fwd.restype = c_int
    _lib.imf_attn_fwd.argtypes = [c_void_p] * 9 + [c_int, c_int, c_int, c_int, c_void_p, c_int64,
                                                   c_int64, c_int64, c_float, c_void_p, c_void_p]


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
    """(o, do | None, lse | None) for (B, L, H, 64) bf16 tensors."""
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
    rc = _lib.imf_attn_fwd(_ptr(ts[0]), _ptr(ts[1]), _ptr(ts[2]),
                           _ptr(ts[3]) if tang else None, _ptr(ts[4]) if tang else None,
                           _ptr(ts[5]) if tang else None, _ptr(o), _ptr(do), _ptr(lse), B, L, H,
                           hd, ctypes.cast(arr, c_void_p), o.stride(0), o.stride(1), o.stride(2),
                           float(scale), _ptr(status_word(q.device)), _stream())
    _check(rc, "imf_attn_fwd")
    return o, do, lse
