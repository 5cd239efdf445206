"""ctypes wrappers for the fused per-token kernels (``csrc/rowops_*.cu``).

All wrappers take raw tensors, allocate outputs, and return them; shapes are
2-D ``[rows, D]`` unless stated.  ``None`` tangents select the primal-only
path of the same kernel.
"""

from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import torch

from . import kernels as K

_lib = K._lib
c_void_p, c_int, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

if K._has("imf_resnorm"):
    _lib.imf_row_grid.restype = c_int
    _lib.imf_row_grid.argtypes = [c_int]
    _lib.imf_resnorm.restype = c_int
    _lib.imf_resnorm.argtypes = [c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    _lib.imf_rmsnorm_seg.restype = c_int
    _lib.imf_rmsnorm_seg.argtypes = [c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int,
                                     c_void_p]
    _lib.imf_qkprep.restype = c_int
    _lib.imf_qkprep.argtypes = [c_void_p] + [c_int] * 8 + [c_float, c_int, c_int, c_void_p]
    if K._has("imf_colsum"):
        _lib.imf_colsum.restype = c_int
        _lib.imf_colsum.argtypes = [c_void_p, c_int, c_void_p]
    _lib.imf_elementwise.restype = c_int
    _lib.imf_elementwise.argtypes = [c_int, c_void_p, c_void_p, c_float, c_float, c_int, c_int,
                                     c_int, c_void_p]

BF16, F32 = torch.bfloat16, torch.float32


def _p(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _ptr_array(ptrs: Sequence[int]):
    return (c_void_p * len(ptrs))(*[c_void_p(x) for x in ptrs])


def _ints(vals: Sequence[int]):
    return (c_int * len(vals))(*vals)


def row_grid(rows: int) -> int:
    return int(_lib.imf_row_grid(rows))


def _chk(rc: int, name: str) -> None:
    K._check(rc, name)
    K.LAUNCHES.count += 1


# ---------------------------------------------------------------- resnorm ---
def resnorm_fwd(res, dres, y, dy, gate, snaps: Sequence[torch.Tensor],
                dsnaps: Sequence[Optional[torch.Tensor]], w, gain, eps: float,
                out_n: torch.Tensor, out_dn: Optional[torch.Tensor],
                out_pfx: Optional[torch.Tensor], out_dpfx: Optional[torch.Tensor]) -> None:
    """n = RMSNorm(remix(res + y*gate, snaps; w)) * gain (+ tangent).
    res/snaps fp32 [rows, D]; y bf16; outputs preallocated."""
    rows, D = out_n.shape
    has_t = out_dn is not None
    ns = len(snaps)
    ptrs = [_p(res), _p(dres), _p(y), _p(dy), _p(gate), _p(w), _p(gain), _p(out_pfx),
            _p(out_dpfx), _p(out_n), _p(out_dn), 0, 0, 0, 0, 0]
    ptrs += [_p(s) for s in snaps] + [_p(s) for s in dsnaps] + [0] * ns
    _chk(_lib.imf_resnorm(_ptr_array(ptrs), ns, rows, D, float(eps), int(has_t), 0, K._stream()),
         "imf_resnorm fwd")


class ColSums:
    """Collects the partial-sum buffers of several row-kernel backward calls and reduces all
    of them in one launch (``imf_colsum``), each straight into its destination: a parameter's
    existing fp32 gradient buffer (accumulated) or a fresh tensor."""

    MAX = 12

    def __init__(self):
        self.items = []        # (partial tensor, column index, D, dst tensor, accumulate)

    def add(self, part: torch.Tensor, col: int, D: int, dst: Optional[torch.Tensor]):
        """``part``: [g, C, D] or [g, D] fp32.  Returns the destination (a new tensor when
        ``dst`` is None)."""
        acc = dst is not None
        if dst is None:
            dst = torch.empty(D, dtype=F32, device=part.device)
        self.items.append((part, col, D, dst, acc))
        return dst

    def flush(self) -> None:
        import numpy as np

        rec = np.dtype([("part", "<u8"), ("dst", "<u8"), ("g", "<i4"), ("D", "<i4"),
                        ("stride", "<i4"), ("acc", "<i4")])
        for i0 in range(0, len(self.items), self.MAX):
            chunk = self.items[i0:i0 + self.MAX]
            host = np.zeros(len(chunk), dtype=rec)
            for i, (part, col, D, dst, acc) in enumerate(chunk):
                stride = part.stride(0)
                host[i] = (part.data_ptr() + 4 * col * D, dst.data_ptr(), part.shape[0], D, stride,
                           int(acc))
            _chk(_lib.imf_colsum(host.ctypes.data_as(ctypes.c_void_p), len(chunk), K._stream()),
                 "imf_colsum")
        self.items = []


def resnorm_bwd(res, y, gate, snaps: Sequence[torch.Tensor], w, gain, eps: float, gn,
                g_pfx_ext, want_g_res: bool = True, raw: bool = False,
                g_snaps_ext: Optional[Sequence[torch.Tensor]] = None):
    """Returns (g_res fp32 | None, g_y bf16 | None, [g_snaps fp32], g_gain, g_w, g_gate);
    with ``raw`` the last three are replaced by the [g, 3, D] partial buffer (columns gain,
    w, gate) for a later ``ColSums`` reduction.  ``g_snaps_ext``: fp32 gradients (one per
    snapshot) that the kernel adds to the snapshot gradients it writes."""
    rows, D = gn.shape
    dev = gn.device
    ns = len(snaps)
    g_res = torch.empty(rows, D, dtype=F32, device=dev) if want_g_res else None
    g_y = torch.empty(rows, D, dtype=BF16, device=dev) if y is not None else None
    g_snaps = [torch.empty(rows, D, dtype=F32, device=dev) for _ in range(ns)]
    partial = torch.empty(row_grid(rows), 3, D, dtype=F32, device=dev)
    ptrs = [_p(res), 0, _p(y), 0, _p(gate), _p(w), _p(gain), 0, 0, 0, 0, _p(gn), _p(g_pfx_ext),
            _p(g_res), _p(g_y), _p(partial)]
    ext = [0] * ns if g_snaps_ext is None else [_p(e) for e in g_snaps_ext[:ns]]
    ptrs += [_p(s) for s in snaps] + ext + [_p(s) for s in g_snaps]
    _chk(_lib.imf_resnorm(_ptr_array(ptrs), ns, rows, D, float(eps), 0, 1, K._stream()),
         "imf_resnorm bwd")
    if raw:
        return g_res, g_y, g_snaps, partial
    col = partial.sum(0)
    return g_res, g_y, g_snaps, col[0], (col[1] if w is not None else None), \
        (col[2] if y is not None else None)


# ----------------------------------------------------------- strided norm ---
def rmsnorm_seg_fwd(segs, rows: int, eps: float, has_t: bool) -> None:
    """segs: list of (x, dx, gain, out, dout, D, ld_x, ld_o) with x/out possibly
    column views of wider buffers (pass the view's data_ptr via tensors)."""
    ptrs, dims = [], []
    for (x, dx, gain, out, dout, D, ld_x, ld_o) in segs:
        ptrs += [_p(x), _p(dx), _p(gain), _p(out), _p(dout), 0, 0, 0]
        dims += [D, ld_x, ld_o]
    _chk(_lib.imf_rmsnorm_seg(_ptr_array(ptrs), _ints(dims), len(segs), rows, float(eps),
                              int(has_t), 0, K._stream()), "imf_rmsnorm_seg fwd")


def rmsnorm_seg_bwd(segs, rows: int, eps: float, raw: bool = False):
    """segs: list of (x, gain, gy, gx, D, ld_x, ld_o); returns [g_gain per seg] (with ``raw``
    the [g, D] partial buffers instead)."""
    ptrs, dims, parts = [], [], []
    g = row_grid(rows)
    for (x, gain, gy, gx, D, ld_x, ld_o) in segs:
        part = torch.empty(g, D, dtype=F32, device=x.device)
        parts.append(part)
        ptrs += [_p(x), 0, _p(gain), 0, 0, _p(gy), _p(gx), _p(part)]
        dims += [D, ld_x, ld_o]
    _chk(_lib.imf_rmsnorm_seg(_ptr_array(ptrs), _ints(dims), len(segs), rows, float(eps), 0, 1,
                              K._stream()), "imf_rmsnorm_seg bwd")
    return parts if raw else [p.sum(0) for p in parts]


# ---------------------------------------------------------------- qk prep ---
def qkprep_fwd(qb, dqb, kvb, dkvb, kr, dkr, cos, sin, qg, kg, q, dq, k, dk, rows, L, H, dn, dr,
               dv, ld_kr, eps) -> None:
    ptrs = [_p(qb), _p(dqb), _p(kvb), _p(dkvb), _p(kr), _p(dkr), _p(cos), _p(sin), _p(qg), _p(kg),
            _p(q), _p(dq), _p(k), _p(dk), 0, 0, 0, 0, 0, 0]
    _chk(_lib.imf_qkprep(_ptr_array(ptrs), rows, L, H, dn, dr, dv, ld_kr, 0, float(eps),
                         int(dq is not None), 0, K._stream()), "imf_qkprep fwd")


def qkprep_bwd(qb, kvb, cos, sin, qg, kg, gq, gk, g_qb, g_kvb, g_kr, rows, L, H, dn, dr, dv,
               ld_gkr, eps, raw: bool = False):
    part = torch.empty(row_grid(rows), 2, dn, dtype=F32, device=qb.device)
    ptrs = [_p(qb), 0, _p(kvb), 0, 0, 0, _p(cos), _p(sin), _p(qg), _p(kg), 0, 0, 0, 0, _p(gq),
            _p(gk), _p(g_qb), _p(g_kvb), _p(g_kr), _p(part)]
    _chk(_lib.imf_qkprep(_ptr_array(ptrs), rows, L, H, dn, dr, dv, 0, ld_gkr, float(eps), 0, 1,
                         K._stream()), "imf_qkprep bwd")
    if raw:
        return part            # [g, 2, dn]: columns q gain, k gain
    col = part.sum(0)
    return col[0], col[1]


# ------------------------------------------------------------ elementwise ---
def _ew(op, ptrs, dims, beta=0.0, lbeta=0.0, has_lb=0, has_t=0, bwd=0, name="ew"):
    _chk(_lib.imf_elementwise(op, _ptr_array(ptrs), _ints(dims), float(beta), float(lbeta),
                              int(has_lb), int(has_t), int(bwd), K._stream()), name)


def outgate_fwd(o, do, g, dg, out, dout, rows, D, ld_o_in, ld_g) -> None:
    ptrs = [_p(o), _p(do), _p(g), _p(dg), 0, 0, 0, _p(out), _p(dout)] + [0] * 7
    _ew(0, ptrs, [rows, D, ld_o_in, ld_g, D, 0, 0], has_t=int(do is not None), name="outgate fwd")


def outgate_bwd(o, g, gout, g_o, g_g, rows, D, ld_o_in, ld_g, ld_go, ld_gg) -> None:
    ptrs = [_p(o), 0, _p(g), 0, 0, 0, 0, 0, 0, 0, 0, _p(gout), 0, _p(g_o), _p(g_g), 0]
    _ew(0, ptrs, [rows, D, ld_o_in, ld_g, D, ld_go, ld_gg], bwd=1, name="outgate bwd")


def situ_fwd(gu, dgu, out, dout, rows, F, beta, lbeta) -> None:
    """gu: [rows, 2F] = [gate | up]; out [rows, F]."""
    up = gu[:, F:]
    dup = None if dgu is None else dgu[:, F:]
    ptrs = [_p(gu), _p(dgu), _p(up), _p(dup), 0, 0, 0, _p(out), _p(dout)] + [0] * 7
    _ew(1, ptrs, [rows, F, 2 * F, 2 * F, F, 0, 0], beta, lbeta or 0.0, int(lbeta is not None),
        int(dgu is not None), 0, "situ fwd")


def situ_bwd(gu, gout, g_gu, rows, F, beta, lbeta) -> None:
    ptrs = [_p(gu), 0, _p(gu[:, F:]), 0, 0, 0, 0, 0, 0, 0, 0, _p(gout), 0, _p(g_gu),
            _p(g_gu[:, F:]), 0]
    _ew(1, ptrs, [rows, F, 2 * F, 2 * F, F, 2 * F, 2 * F], beta, lbeta or 0.0,
        int(lbeta is not None), 0, 1, "situ bwd")


def scale_add_fwd(res, dres, y, dy, gate, out, dout, rows, D) -> None:
    ptrs = [_p(y), _p(dy), 0, 0, _p(res), _p(dres), _p(gate), 0, 0, _p(out), _p(dout)] + [0] * 5
    _ew(2, ptrs, [rows, D, D, D, D, 0, 0], has_t=int(dy is not None), name="scale_add fwd")


def scale_add_bwd(y, gate, g_out, rows, D, raw: bool = False):
    """Returns (g_y bf16, g_gate fp32 -- the [g, D] partial buffer with ``raw``); the gradient
    of `res` is g_out itself."""
    g_y = torch.empty(rows, D, dtype=BF16, device=y.device)
    part = torch.empty(row_grid(rows), D, dtype=F32, device=y.device)
    ptrs = [_p(y), 0, 0, 0, 0, 0, _p(gate), 0, 0, 0, 0, 0, _p(g_out), _p(g_y), 0, _p(part)]
    _ew(2, ptrs, [rows, D, D, D, D, D, D], bwd=1, name="scale_add bwd")
    return g_y, (part if raw else part.sum(0))
