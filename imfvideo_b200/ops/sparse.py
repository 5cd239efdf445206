"""Wrappers for the block-sparse attention kernels (``csrc/attn_sparse.cu``):
per-block INT8 quantiser, query-tile LUT construction, forward (+ tangent),
and ``SparseCore``, the attention core that plugs SLA2 / cube attention into
the fused transformer-block node (``ops/block.py``)."""

from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch

from . import kernels as K

_lib = K._lib
vp, ci, cf, c64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_int64

if K._has("imf_attn_sparse_fwd"):
    _lib.imf_quantize_blocks.restype = ci
    _lib.imf_quantize_blocks.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, c64, c64, c64, vp]
    _lib.imf_attn_sparse_fwd.restype = ci
    _lib.imf_attn_sparse_fwd.argtypes = [vp] * 16 + [ci] * 5 + [vp, c64, c64, c64, cf, ci, ci, vp, vp]


_HAS_MANY = K._has("imf_quantize_blocks_many")
if _HAS_MANY:
    _lib.imf_quantize_blocks_many.restype = ci
    _lib.imf_quantize_blocks_many.argtypes = [vp, vp, ci, ci, ci, ci, vp]

if K._has("imf_build_tile_lut"):
    _lib.imf_build_tile_lut.restype = ci
    _lib.imf_build_tile_lut.argtypes = [vp] * 6 + [ci] * 7 + [vp]
    _lib.imf_build_kv_lists.restype = ci
    _lib.imf_build_kv_lists.argtypes = [vp] * 5 + [ci] * 5 + [vp]


ROUTER_KERNELS = K._has("imf_route_topk")
if ROUTER_KERNELS:
    _lib.imf_pool_blocks.restype = ci
    _lib.imf_pool_blocks.argtypes = [vp, vp] + [ci] * 5 + [c64] * 3 + [vp]
    _lib.imf_route_topk.restype = ci
    _lib.imf_route_topk.argtypes = [vp] * 6 + [ci] * 8 + [cf, vp]


def pool_blocks(x: torch.Tensor, block: int, nb: Optional[int] = None) -> torch.Tensor:
    """Means of the first ``nb`` blocks of ``block`` rows (ragged last block: mean of its
    valid rows).  x: (B, H, L, 64) bf16 view with a contiguous last dim -> (B, H, nb, 64) fp32."""
    B, H, L, D = x.shape
    assert D == 64 and x.dtype == torch.bfloat16 and x.stride(3) == 1
    nb = -(-L // block) if nb is None else nb
    out = torch.empty(B, H, nb, D, dtype=torch.float32, device=x.device)
    K._check(_lib.imf_pool_blocks(K._ptr(x), K._ptr(out), B, min(L, nb * block), H, block, nb,
                                  x.stride(0), x.stride(2), x.stride(1), K._stream()),
             "imf_pool_blocks")
    K.LAUNCHES.count += 1
    return out


def route_topk(qb: torch.Tensor, kb: torch.Tensor, T: int, proj_q: Optional[torch.Tensor] = None,
               proj_k: Optional[torch.Tensor] = None, n_keys: Optional[int] = None,
               n_tail: int = 0, tail0: int = 0, want_scores: bool = False):
    """Hard top-``T`` of the projected block scores (one launch).  qb (B, H, Mb, 64), kb
    (B, H, Nkb, 64) fp32 pooled blocks; the first ``n_keys`` key blocks are candidates;
    ``n_tail`` always-attended block ids ``tail0, tail0 + 1, ...`` are appended to every row.
    Returns sel (B, H, Mb, T + n_tail) int32 (ascending within the two groups of the
    selection) and, on request, the scores (B, H, Mb, n_keys) fp32."""
    B, H, Mb, D = qb.shape
    Nkb = kb.shape[2]
    Nk = Nkb if n_keys is None else n_keys
    assert D == 64 and qb.dtype == kb.dtype == torch.float32
    qb, kb = qb.contiguous(), kb.contiguous()
    pq = None if proj_q is None else proj_q.detach().float().contiguous()
    pk = None if proj_k is None else proj_k.detach().float().contiguous()
    sel = torch.empty(B, H, Mb, T + n_tail, dtype=torch.int32, device=qb.device)
    sc = torch.empty(B, H, Mb, Nk, dtype=torch.float32, device=qb.device) if want_scores else None
    K._check(_lib.imf_route_topk(K._ptr(qb), K._ptr(kb), K._ptr(pq), K._ptr(pk), K._ptr(sel),
                                 K._ptr(sc), B, H, Mb, Nkb, Nk, T, n_tail, tail0,
                                 float(D) ** -0.5, K._stream()), "imf_route_topk")
    K.LAUNCHES.count += 1
    return (sel, sc) if want_scores else sel


def route_tables(sel: torch.Tensor, qblk: int, L: int):
    """Device-built routing tables from the selection ``sel`` (B, H, Mb, T): the per-tile
    key-block lists of ``build_tile_lut`` (ascending, -1 padded), their flags, the entry
    counts, and the maps the inverted lists are made from: one uint8 tensor
    (3, B, H, n_kvt, n_mt) whose planes 0-1 are a uint16 rank matrix (for a live
    (K/V tile, query tile) pair, how many higher K/V tiles attend the same query tile: the
    backward's place in the fixed order of dQ additions) and whose plane 2 is the nibble
    matrix of live 64 x 64 quadrants.  One launch, no host synchronisation."""
    B, H, Mb, T = sel.shape
    sel = sel.to(torch.int32).contiguous()
    n_mt = -(-L // 128)
    tmax = T * (128 // qblk)
    dev = sel.device
    lut = torch.empty(B, H, n_mt, tmax, dtype=torch.int32, device=dev)
    flags = torch.empty(B, H, n_mt, tmax, dtype=torch.uint8, device=dev)
    cnt = torch.empty(B, H, n_mt, dtype=torch.int32, device=dev)
    maps = torch.empty(3, B, H, n_mt, n_mt, dtype=torch.uint8, device=dev)
    K._check(_lib.imf_build_tile_lut(K._ptr(sel), K._ptr(lut), K._ptr(flags), K._ptr(cnt),
                                     K._ptr(maps[2]), K._ptr(maps), B, H, Mb, T, qblk, L, tmax,
                                     K._stream()),
             "imf_build_tile_lut")
    K.LAUNCHES.count += 1
    return lut, flags, cnt, maps


def kv_lists(maps: torch.Tensor, want_rank: bool = False):
    """Inverted lists for the backward kernel from the maps of ``route_tables`` (or a bare
    (B, H, n_kvt, n_mt) nibble matrix): (qlist int32 (B,H,n_kvt,n_mt) padded with -1, qflags
    uint8) and, with ``want_rank``, qrank int16 (the entry's place in the fixed order of dQ
    additions; None for a bare nibble matrix).  The list stride is the static bound n_mt, so
    no host read of the longest list is needed."""
    packed = maps.dim() == 5
    fm = maps[2] if packed else maps
    B, H, n_kvt, n_mt = fm.shape
    qlist = torch.empty(B, H, n_kvt, n_mt, dtype=torch.int32, device=fm.device)
    qflags = torch.empty(B, H, n_kvt, n_mt, dtype=torch.uint8, device=fm.device)
    qrank = (torch.empty(B, H, n_kvt, n_mt, dtype=torch.int16, device=fm.device)
             if packed and want_rank else None)
    K._check(_lib.imf_build_kv_lists(K._ptr(fm), K._ptr(maps) if qrank is not None else None,
                                     K._ptr(qlist), K._ptr(qflags), K._ptr(qrank), B, H, n_kvt,
                                     n_mt, n_mt, K._stream()), "imf_build_kv_lists")
    K.LAUNCHES.count += 1
    return (qlist, qflags, qrank) if want_rank else (qlist, qflags)


def quantize_blocks(x: torch.Tensor, block: int, want_q: bool = True, want_fq: bool = False):
    """x: (B, L, H, 64) bf16 -> (int8 (B,L,H,64) | None, scales (B,H,nblk) fp32,
    de-quantised bf16 copy | None)."""
    B, L, H, D = x.shape
    assert D == 64 and x.dtype == torch.bfloat16 and x.stride(3) == 1
    nb = -(-L // block)
    xq = torch.empty(B, L, H, D, dtype=torch.int8, device=x.device) if want_q else None
    xs = torch.empty(B, H, nb, dtype=torch.float32, device=x.device)
    xf = torch.empty(B, L, H, D, dtype=torch.bfloat16, device=x.device) if want_fq else None
    K._check(_lib.imf_quantize_blocks(K._ptr(x), K._ptr(xq), K._ptr(xs), K._ptr(xf), B, L, H, block,
                                      x.stride(0), x.stride(1), x.stride(2), K._stream()),
             "imf_quantize_blocks")
    K.LAUNCHES.count += 1
    return xq, xs, xf


def quantize_blocks_many(items, block: int = 64):
    """``quantize_blocks`` for up to three tensors of one shape -- the q, k, v of an attention
    call -- in one launch.  items: [(x, want_q, want_fq)]; returns [(xq, xs, xf)].  Falls back
    to one launch per tensor when the shapes differ, the blocks are not 64 rows, or a tensor's
    rows are not 16-byte aligned."""
    xs_ = [K._tma_ok(x) for x, _, _ in items]
    same = all(x.shape == xs_[0].shape and x.dtype == torch.bfloat16 and x.stride(3) == 1
               and x.data_ptr() % 16 == 0 and all(st % 8 == 0 for st in x.stride()[:3])
               for x in xs_)
    if not (_HAS_MANY and block == 64 and 1 < len(items) <= 3 and same and xs_[0].shape[3] == 64):
        return [quantize_blocks(x, block, want_q=wq, want_fq=wf) for x, (_, wq, wf) in zip(xs_, items)]
    B, L, H, D = xs_[0].shape
    nb = -(-L // 64)
    dev = xs_[0].device
    outs, ptrs, strides = [], [], []
    for x, (_, wq, wf) in zip(xs_, items):
        xq = torch.empty(B, L, H, D, dtype=torch.int8, device=dev) if wq else None
        sc = torch.empty(B, H, nb, dtype=torch.float32, device=dev)
        xf = torch.empty(B, L, H, D, dtype=torch.bfloat16, device=dev) if wf else None
        outs.append((xq, sc, xf))
        ptrs += [x.data_ptr(), 0 if xq is None else xq.data_ptr(), sc.data_ptr(),
                 0 if xf is None else xf.data_ptr()]
        strides += [x.stride(0), x.stride(1), x.stride(2)]
    parr = (ctypes.c_void_p * len(ptrs))(*ptrs)
    sarr = (c64 * len(strides))(*strides)
    K._check(_lib.imf_quantize_blocks_many(parr, sarr, len(items), B, L, H, K._stream()),
             "imf_quantize_blocks_many")
    K.LAUNCHES.count += 1
    return outs


def build_tile_lut(sel: torch.Tensor, qblk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-128-row query tile list of 64-key blocks from the per-routing-block
    selection ``sel`` (B, H, Mb, T).  qblk 128: one routing block per tile.
    qblk 64: a tile holds two routing blocks; the list is their union and the
    flags say which half attends each entry (bit0 rows 0-63, bit1 rows 64-127).
    Returns (lut int32 (B,H,n_mt,tmax) padded with -1, flags uint8)."""
    B, H, Mb, T = sel.shape
    sel = sel.to(torch.int32)
    if qblk == 128:
        return sel.contiguous(), torch.full(sel.shape, 3, dtype=torch.uint8, device=sel.device)
    n_mt = (Mb + 1) // 2
    if Mb % 2:
        sel = torch.cat([sel, torch.full((B, H, 1, T), -1, dtype=torch.int32, device=sel.device)], 2)
    pair = sel.view(B, H, n_mt, 2 * T)
    fl = torch.cat([torch.ones(T, dtype=torch.int32, device=sel.device),
                    torch.full((T,), 2, dtype=torch.int32, device=sel.device)]).expand(B, H, n_mt, 2 * T)
    big = torch.iinfo(torch.int32).max
    ids = torch.where(pair < 0, torch.full_like(pair, big), pair)
    ids, order = ids.sort(dim=-1)
    fl = torch.gather(fl, -1, order)
    dup = torch.zeros_like(ids, dtype=torch.bool)
    dup[..., 1:] = (ids[..., 1:] == ids[..., :-1]) & (ids[..., 1:] != big)
    # a block selected by both halves appears twice in a row: merge the flags into the first
    fl_next = torch.zeros_like(fl)
    fl_next[..., :-1] = torch.where(dup[..., 1:], fl[..., 1:], torch.zeros_like(fl[..., 1:]))
    fl = fl | fl_next
    ids = torch.where(dup, torch.full_like(ids, big), ids)
    ids, order = ids.sort(dim=-1)
    fl = torch.gather(fl, -1, order)
    lut = torch.where(ids == big, torch.full_like(ids, -1), ids)
    return lut.contiguous(), fl.to(torch.uint8).contiguous()


def sparse_fwd(q, k, v, dq, dk, dv, lut, flags, qblk: int, int8: bool, quant_p: bool,
               need_lse: bool = True, scale: Optional[float] = None,
               cnt: Optional[torch.Tensor] = None):
    """Block-sparse softmax branch: (o_s, do_s | None, lse | None).
    q, k, v (+ tangents): (B, L, H, 64) bf16, token order = routing order."""
    B, L, H, D = q.shape
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    tang = dq is not None
    q8 = k8 = qs = ks = None
    vv = K._tma_ok(v)
    if int8 and qblk == 64:
        (q8, qs, _), (k8, ks, _), (_, _, vv) = quantize_blocks_many(
            [(q, True, False), (k, True, False), (vv, False, True)])
    elif int8:
        q8, qs, _ = quantize_blocks(K._tma_ok(q), qblk)
        k8, ks, _ = quantize_blocks(K._tma_ok(k), 64)
        _, _, vv = quantize_blocks(vv, 64, want_q=False, want_fq=True)
    ts = [K._tma_ok(q), K._tma_ok(k), vv]
    if tang:
        ts += [K._tma_ok(dq), K._tma_ok(dk), K._tma_ok(dv)]
    strides = []
    for t in ts:
        strides += [t.stride(0), t.stride(1), t.stride(2)]
    arr = (c64 * 18)(*(strides + [0] * (18 - len(strides))))
    o = torch.empty(B, L, H, D, dtype=torch.bfloat16, device=q.device)
    do = torch.empty_like(o) if tang else None
    lse = torch.empty(B, H, L, dtype=torch.float32, device=q.device) if need_lse else None
    need_qk = tang or not int8
    if cnt is None:     # entries per list = position of the first -1
        cnt = (lut >= 0).to(torch.int32).cumprod(-1).sum(-1, dtype=torch.int32).contiguous()
    rc = _lib.imf_attn_sparse_fwd(
        K._ptr(q8), K._ptr(k8), K._ptr(qs), K._ptr(ks),
        K._ptr(ts[0]) if need_qk else None, K._ptr(ts[1]) if need_qk else None, K._ptr(ts[2]),
        K._ptr(ts[3]) if tang else None, K._ptr(ts[4]) if tang else None,
        K._ptr(ts[5]) if tang else None, K._ptr(lut), K._ptr(flags), K._ptr(cnt), K._ptr(o),
        K._ptr(do),
        K._ptr(lse), B, L, H, lut.shape[-1], qblk, ctypes.cast(arr, vp), o.stride(0), o.stride(1),
        o.stride(2), float(scale), int(quant_p), int(int8), K._ptr(K.status_word(q.device)),
        K._stream())
    K._check(rc, "imf_attn_sparse_fwd")
    K.LAUNCHES.count += 1
    return o, do, lse


def build_kv_lists(lut: torch.Tensor, flags: torch.Tensor, L: int):
    """Invert the query-tile LUT for the backward: for every 128-row K/V tile
    (two 64-key blocks) the list of 128-row query tiles that attend it, with 4
    flag bits per entry (bit = kv half * 2 + q half).  Returns
    (qlist int32 (B,H,n_kvt,qmax) padded with -1, qflags uint8)."""
    B, H, n_mt, tmax = lut.shape
    n_kvt = -(-L // 128)
    valid = lut >= 0
    kb = torch.where(valid, lut, torch.zeros_like(lut)).long()
    val = (flags.to(torch.int32) << (2 * (kb % 2)).to(torch.int32)) * valid.to(torch.int32)
    F = torch.zeros(B, H, n_kvt, n_mt, dtype=torch.int32, device=lut.device)
    mt = torch.arange(n_mt, device=lut.device).view(1, 1, n_mt, 1).expand(B, H, n_mt, tmax)
    flat = (kb // 2) * n_mt + mt                        # index into (n_kvt * n_mt)
    F.view(B, H, -1).scatter_add_(2, flat.reshape(B, H, -1), val.reshape(B, H, -1))
    live = F > 0
    qmax = int(live.sum(-1).max().item())
    order = torch.argsort((~live).to(torch.int8), dim=-1, stable=True)[..., :qmax]
    qf = torch.gather(F, -1, order)
    ql = torch.where(qf > 0, order.to(torch.int32), torch.full_like(order, -1, dtype=torch.int32))
    return ql.contiguous(), qf.to(torch.uint8).contiguous()
