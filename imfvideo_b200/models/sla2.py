"""SLA2 sparse-linear attention: 1-D block form and 3-D "cube" tile form with
INT8 quantisation-aware training, as attention plug-ins on dual numbers.

    O   = a * O_s + (1 - a) * O_l
    O_s = softmax(Q K^T / sqrt(d) restricted to the routed key blocks) V
    O_l = (phi(Q) phi(K)^T restricted to the complement blocks) V / rowsum
    a   = sigmoid(alpha_logit)[head, query block],  phi = softmax over channels

Semantics follow the reference (``models/sla2_vendor/core.py:78-180``,
``models/sla2_vendor/router.py:22-90``, ``models/sla2_attention.py:23-61``,
``models/mla_video_sparse_jvp.py:61-91,268-295,457-498``,
``models/sla2_cube_qat.py:295-439``): learnable router with identity-
initialised projections and hard top-k (SoftTop-k for router training),
per-(head, query-block) mixing logits, always-attended prefix tail for cube
tiles, symmetric per-block INT8 fake quantisation (scale = amax / 127, round
half away from zero) with a straight-through gradient.

The formulas here are the CPU path and the oracle.  They never materialise an
(L, L) matrix: selected key blocks are gathered (O(L * topk * bk)) and the
complement goes through per-block phi(K)^T V states.  On CUDA the sparse
branch runs in the block-sparse tcgen05 kernels (``ops/sparse.py``).
"""

from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.dual import Dual

Tensor = torch.Tensor
EPS_LINEAR = 1e-5


# ------------------------------------------------------------- geometry ---
def tile_permutation(grid, tile, prefix_len: int, device=None):
    """Index maps between model order ``[prefix | patches, t-major]`` and tile
    order ``[patches grouped by 3-D tile | prefix]``.  Returns (perm, inv, Np)
    with ``tile_tokens = model_tokens[perm]`` and ``model = tile[inv]``."""
    T, Hh, Ww = grid
    tt, th, tw = tile
    assert T % tt == 0 and Hh % th == 0 and Ww % tw == 0, (grid, tile)
    idx = torch.arange(T * Hh * Ww, device=device).view(T // tt, tt, Hh // th, th, Ww // tw, tw)
    idx = idx.permute(0, 2, 4, 1, 3, 5).reshape(-1) + prefix_len
    perm = torch.cat([idx, torch.arange(prefix_len, device=device)])
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), device=device)
    return perm, inv, (T // tt) * (Hh // th) * (Ww // tw)


def _router_kernels_ok(q: Tensor, k: Tensor) -> bool:
    """Pooling + top-k on the kernel library: CUDA bf16 (B, H, L, 64) views with a contiguous
    last dim and at most 4096 key blocks' worth of candidates."""
    if not (q.is_cuda and q.dtype == k.dtype == torch.bfloat16 and q.shape[-1] == 64):
        return False
    if q.stride(-1) != 1 or k.stride(-1) != 1 or torch._C._are_functorch_transforms_active():
        return False
    if k.shape[2] > 4096 * 64:          # the top-k kernel holds one score per key block in smem
        return False
    try:
        from ..ops import sparse as SP
        return SP.ROUTER_KERNELS
    except Exception:
        return False


def block_mean(x: Tensor, block: int) -> Tensor:
    """(B, H, L, D) -> (B, H, ceil(L / block), D) means (ragged last block)."""
    B, H, L, D = x.shape
    nb = -(-L // block)
    pad = nb * block - L
    xf = F.pad(x.float(), (0, 0, 0, pad)).reshape(B, H, nb, block, D).sum(3)
    cnt = torch.full((nb,), float(block), device=x.device)
    cnt[-1] = block - pad
    return xf / cnt.view(1, 1, nb, 1)


# --------------------------------------------------------------- router ---
def soft_topk(pc: Tensor, k_frac: float, tau: float = 0.1, n_iters: int = 30) -> Tensor:
    """sigmoid(pc / tau + lambda_row) with every row summing to k_frac * Nb
    (bisection on lambda; lambda carries no gradient)."""
    x = pc.float() / tau
    target = k_frac * pc.shape[-1]
    lo = torch.full(pc.shape[:-1], -1e4, device=pc.device)
    hi = torch.full(pc.shape[:-1], 1e4, device=pc.device)
    with torch.no_grad():
        for _ in range(n_iters):
            mid = 0.5 * (lo + hi)
            big = torch.sigmoid(x + mid[..., None]).sum(-1) > target
            hi = torch.where(big, mid, hi)
            lo = torch.where(big, lo, mid)
        lam = 0.5 * (lo + hi)
    return torch.sigmoid(x + lam[..., None])


class Router(nn.Module):
    """Pooled, projected block scores and the routed block table."""

    def __init__(self, head_dim: int, bq: int = 128, bk: int = 64, tau: float = 0.1,
                 learnable: bool = True):
        super().__init__()
        self.bq, self.bk, self.tau, self.learnable = bq, bk, tau, learnable
        self.proj_q = nn.Linear(head_dim, head_dim, bias=False)
        self.proj_k = nn.Linear(head_dim, head_dim, bias=False)
        with torch.no_grad():
            self.proj_q.weight.copy_(torch.eye(head_dim))
            self.proj_k.weight.copy_(torch.eye(head_dim))
        if not learnable:
            for p in self.parameters():
                p.requires_grad_(False)

    def scores(self, q: Tensor, k: Tensor) -> Tensor:
        """(B, H, L, D) -> (B, H, Mb, Nb) fp32; keys are centred (smooth-k)."""
        qb = block_mean(q, self.bq)
        kb = block_mean(k.float() - k.float().mean(-2, keepdim=True), self.bk)
        if self.learnable:
            qb, kb = self.proj_q(qb), self.proj_k(kb)
        return (qb @ kb.transpose(-1, -2)) * (q.shape[-1] ** -0.5)

    def forward(self, q, k, k_frac: float, soft: bool = False, need_mask: bool = True):
        if not soft and not need_mask and _router_kernels_ok(q, k):
            from ..ops import sparse as SP

            nb = -(-k.shape[2] // self.bk)
            topk = max(1, min(nb, int(k_frac * nb)))
            pq, pk = ((self.proj_q.weight, self.proj_k.weight) if self.learnable
                      else (None, None))
            lut = SP.route_topk(SP.pool_blocks(q, self.bq), SP.pool_blocks(k, self.bk), topk,
                                pq, pk)
            return None, lut, topk, None
        pc = self.scores(q, k)
        nb = pc.shape[-1]
        topk = max(1, min(nb, int(k_frac * nb)))
        lut = torch.topk(pc, topk, dim=-1, sorted=False).indices.to(torch.int32).contiguous()
        if soft:
            return soft_topk(pc, k_frac, self.tau), lut, topk, pc
        hard = (torch.zeros_like(pc, dtype=torch.int8).scatter_(-1, lut.long(), 1)
                if need_mask else pc)
        return hard, lut, topk, pc


def route_tiles(q: Tensor, k: Tensor, topk_frac: float, Np: int, E: int, prefix_len: int,
                proj_q: Optional[Tensor] = None, proj_k: Optional[Tensor] = None,
                n_tail: int = 0):
    """Hard top-k over pooled (projected) tile scores.  q, k tile-major
    (B, H, L, D); returns lut (B, H, Mb, T + n_tail) of VIDEO tile ids (followed by the
    always-attended tail blocks Np, Np + 1, ...) and T.  The mean
    key subtraction of the 1-D router is a per-row constant here and cannot
    change a hard top-k, so it is omitted."""
    T = max(1, min(Np, int(topk_frac * Np)))
    if _router_kernels_ok(q, k):
        from ..ops import sparse as SP

        lut = SP.route_topk(SP.pool_blocks(q, E), SP.pool_blocks(k, E, Np), T, proj_q, proj_k,
                            n_tail=n_tail, tail0=Np)
        return lut, T
    qb = block_mean(q, E)                                   # (B,H,Mb,D) incl. prefix tail blocks
    kb = block_mean(k[:, :, :Np * E], E)                    # (B,H,Np,D)
    if proj_q is not None:
        qb = qb @ proj_q.t().to(qb.dtype)
    if proj_k is not None:
        kb = kb @ proj_k.t().to(kb.dtype)
    pc = (qb @ kb.transpose(-1, -2)) * (q.shape[-1] ** -0.5)
    lut = torch.topk(pc, T, dim=-1, sorted=False).indices.to(torch.int32)
    if n_tail:
        tail = torch.arange(Np, Np + n_tail, device=q.device, dtype=lut.dtype)
        lut = torch.cat([lut, tail.view(1, 1, 1, -1).expand(*lut.shape[:3], -1)], dim=-1)
    return lut.contiguous(), T


# ---------------------------------------------------------- quantisation ---
def _round_ste(x: Tensor) -> Tensor:
    """Round half away from zero; identity for gradients and tangents."""
    r = torch.sign(x) * torch.floor(x.abs() + 0.5)
    return x + (r - x).detach()


def fake_quant_blocks(x: Tensor, block: int) -> Tensor:
    """Symmetric per-(batch, head, token-block) INT8 fake quantisation with a
    straight-through gradient/tangent.  x: (B, H, L, D)."""
    B, H, L, D = x.shape
    nb = -(-L // block)
    pad = nb * block - L
    xp = F.pad(x.float(), (0, 0, 0, pad)).reshape(B, H, nb, block * D)
    s = (xp.detach().abs().amax(-1, keepdim=True) / 127.0 + 1e-12)
    y = _round_ste(xp / s).clamp(-127, 127) * s
    return y.reshape(B, H, nb * block, D)[:, :, :L].to(x.dtype)


def quantize_blocks(x: Tensor, block: int) -> Tuple[Tensor, Tensor]:
    """(int8 values (B,H,L,D), fp32 scales (B,H,Nb)); reference ``quantize_qkv``."""
    B, H, L, D = x.shape
    nb = -(-L // block)
    pad = nb * block - L
    xp = F.pad(x.float(), (0, 0, 0, pad)).reshape(B, H, nb, block * D)
    s = xp.abs().amax(-1) / 127.0 + 1e-12
    xq = (torch.sign(xp) * torch.floor((xp / s[..., None]).abs() + 0.5)).clamp(-127, 127)
    return xq.reshape(B, H, nb * block, D)[:, :, :L].to(torch.int8), s


# -------------------------------------------------- block sparse + linear ---
def sparse_linear_attention(q: Tensor, k: Tensor, v: Tensor, sel: Tensor, bq: int, bk: int,
                            alpha_rows: Tensor, n_comp_blocks: Optional[int] = None,
                            int8: bool = False, return_parts: bool = False):
    """O = a O_s + (1 - a) O_l without forming an (L, L) matrix.

    q, k, v: (B, H, L, D);  sel: (B, H, Mb, T) selected key-block ids per query
    block (duplicates not allowed);  alpha_rows: (H, L) mixing ratio per row.
    n_comp_blocks: only key blocks < this take part in the linear complement
    (cube attention excludes the always-attended prefix tail blocks).
    int8: fake-quantise Q (per query block) and K, V (per key block) and P
    (x127) in the sparse branch, straight-through.
    """
    B, H, L, D = q.shape
    Mb, Nb = -(-L // bq), -(-L // bk)
    assert sel.shape[2] == Mb, (sel.shape, Mb)
    T = sel.shape[-1]
    scale = D ** -0.5
    qs, ks, vs = q, k, v
    if int8:
        qs, ks, vs = fake_quant_blocks(q, bq), fake_quant_blocks(k, bk), fake_quant_blocks(v, bk)
    pad_q, pad_k = Mb * bq - L, Nb * bk - L
    padq = lambda t: F.pad(t.float(), (0, 0, 0, pad_q)).reshape(B, H, Mb, bq, D)
    padk = lambda t: F.pad(t.float(), (0, 0, 0, pad_k)).reshape(B, H, Nb, bk, D)
    qb, kb, vb = padq(qs), padk(ks), padk(vs)
    idx = sel.long()
    gather = lambda t: torch.gather(
        t.unsqueeze(2).expand(B, H, Mb, Nb, bk, D), 3,
        idx.view(B, H, Mb, T, 1, 1).expand(B, H, Mb, T, bk, D))
    kg, vg = gather(kb), gather(vb)                           # (B,H,Mb,T,bk,D)
    s = torch.einsum("bhmqd,bhmtkd->bhmqtk", qb, kg) * scale
    key_pos = idx.unsqueeze(-1) * bk + torch.arange(bk, device=q.device)    # (B,H,Mb,T,bk)
    valid = (key_pos < L).unsqueeze(3)                        # (B,H,Mb,1,T,bk)
    s = s.masked_fill(~valid, float("-inf")).flatten(-2)      # (B,H,Mb,bq,T*bk)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    if int8:
        # the kernel quantises exp2(s - running max) in [0, 1] by x127; relative to the
        # final normalised p that is the same grid scaled by the row max of p
        pm = p.detach().amax(-1, keepdim=True).clamp_min(1e-30)
        p = _round_ste(p / pm * 127.0) / 127.0 * pm
    o_s = torch.einsum("bhmqk,bhmkd->bhmqd", p, vg.flatten(3, 4)).reshape(B, H, Mb * bq, D)[:, :, :L]

    o_l = linear_branch(q, k, v, sel, bq, bk, n_comp_blocks)
    a = alpha_rows.view(1, H, L, 1).float()
    out = a * o_s + (1.0 - a) * o_l
    if return_parts:
        return out, o_s, o_l, lse.reshape(B, H, Mb * bq)[:, :, :L]
    return out


def linear_branch(q: Tensor, k: Tensor, v: Tensor, sel: Tensor, bq: int, bk: int,
                  n_comp_blocks: Optional[int] = None) -> Tensor:
    """Complement linear attention through per-key-block states
    H_j = phi(K_j)^T V_j, z_j = sum phi(K_j): for query block i the complement
    state is (sum_j H_j) - sum_{j in sel(i)} H_j, formed with one small
    (Mb x Nb) mask matmul.  (B, H, L, D) fp32 in and out."""
    B, H, L, D = q.shape
    Mb, Nb = -(-L // bq), -(-L // bk)
    pad_q, pad_k = Mb * bq - L, Nb * bk - L
    phi_q = F.softmax(q.float(), dim=-1)
    phi_k = F.softmax(k.float(), dim=-1)
    nc = Nb if n_comp_blocks is None else n_comp_blocks
    kmask = (torch.arange(Nb * bk, device=q.device) < min(L, nc * bk)).view(1, 1, Nb, bk, 1)
    pkb = F.pad(phi_k, (0, 0, 0, pad_k)).reshape(B, H, Nb, bk, D) * kmask
    vb = F.pad(v.float(), (0, 0, 0, pad_k)).reshape(B, H, Nb, bk, D)
    Hs = torch.einsum("bhnkd,bhnke->bhnde", pkb, vb)          # (B,H,Nb,D,D)
    zs = pkb.sum(3)                                           # (B,H,Nb,D)
    msel = torch.zeros(B, H, Mb, Nb, device=q.device).scatter_(-1, sel.long(), 1.0)
    Hc = Hs.sum(2, keepdim=True) - torch.einsum("bhmn,bhnde->bhmde", msel, Hs)
    zc = zs.sum(2, keepdim=True) - torch.einsum("bhmn,bhnd->bhmd", msel, zs)
    pq = F.pad(phi_q, (0, 0, 0, pad_q)).reshape(B, H, Mb, bq, D)
    num = torch.einsum("bhmqd,bhmde->bhmqe", pq, Hc)
    den = torch.einsum("bhmqd,bhmd->bhmq", pq, zc).unsqueeze(-1) + EPS_LINEAR
    return (num / den).reshape(B, H, Mb * bq, D)[:, :, :L]


def expand_mask(mc: Tensor, bq: int, bk: int, L: int) -> Tensor:
    return mc.repeat_interleave(bq, dim=-2).repeat_interleave(bk, dim=-1)[..., :L, :L]


def sla2_dense(q, k, v, mc, alpha, bq: int, bk: int, comp_mask: Optional[Tensor] = None):
    """Dense fp32 reference (small L only).  mc: (B, H, Mb, Nb) hard {0,1}
    int8 or soft [0,1];  alpha: (Mb,) or (H, Mb);  comp_mask: optional
    (B, H, Mb, Nb) override of the complement (default 1 - mc)."""
    B, H, L, D = q.shape
    m = expand_mask(mc.float(), bq, bk, L)
    s = (q.float() @ k.float().transpose(-1, -2)) * D ** -0.5
    if mc.dtype == torch.int8 or mc.dtype == torch.bool:
        p = torch.softmax(s.masked_fill(m <= 0, float("-inf")), dim=-1)
    else:
        p = torch.softmax(s + torch.log(m + 1e-9), dim=-1)
    o_s = p @ v.float()
    qphi, kphi = F.softmax(q.float(), -1), F.softmax(k.float(), -1)
    comp = (1.0 - m) if comp_mask is None else expand_mask(comp_mask.float(), bq, bk, L)
    w = (qphi @ kphi.transpose(-1, -2)) * comp
    o_l = (w @ v.float()) / (w.sum(-1, keepdim=True) + EPS_LINEAR)
    a = alpha if alpha.dim() == 2 else alpha.view(1, -1).expand(H, -1)
    a = a.repeat_interleave(bq, dim=-1)[:, :L].view(1, H, L, 1)
    return a * o_s + (1.0 - a) * o_l


def full_attention(q, k, v):
    s = (q.float() @ k.float().transpose(-1, -2)) * q.shape[-1] ** -0.5
    return torch.softmax(s, dim=-1) @ v.float()


# --------------------------------------------------------------- modules ---
def _dual_apply(fn, q: Dual, k: Dual, v: Dual) -> Dual:
    """Primal with its autograd graph; tangent by forward-mode AD of the same
    formulas (detached)."""
    p = fn(q.p, k.p, v.p)
    t = None
    if q.t is not None:
        with torch.no_grad():
            _, t = torch.func.jvp(fn, (q.p.detach(), k.p.detach(), v.p.detach()),
                                  (q.t, k.t, v.t))
    return Dual(p, t)


class SLA2(nn.Module):
    """1-D block SLA2 on (B, H, L, D) tensors (reference ``SLA2`` class)."""

    def __init__(self, head_dim, topk=0.03, bq=128, bk=64, tau=0.1, use_int8=False,
                 learnable_router=True, alpha_init=0.9):
        super().__init__()
        self.topk, self.bq, self.bk, self.use_int8 = topk, bq, bk, use_int8
        self.router = Router(head_dim, bq=bq, bk=bk, tau=tau, learnable=learnable_router)
        self._alpha_init = alpha_init
        self.alpha_logit: Optional[nn.Parameter] = None

    def _get_alpha(self, n_heads, n_qblocks, device) -> Tensor:
        if self.alpha_logit is None or tuple(self.alpha_logit.shape) != (n_heads, n_qblocks):
            init = math.log(self._alpha_init / (1 - self._alpha_init))
            self.alpha_logit = nn.Parameter(torch.full((n_heads, n_qblocks), init, device=device))
        return torch.sigmoid(self.alpha_logit)

    def forward(self, q, k, v, return_sparsity=False, soft_routing=False):
        B, H, L, D = q.shape
        with torch.set_grad_enabled(soft_routing and torch.is_grad_enabled()):
            mask, lut, topk, _pc = self.router(q.detach() if not soft_routing else q,
                                               k.detach() if not soft_routing else k,
                                               self.topk, soft=soft_routing)
        alpha = self._get_alpha(H, -(-L // self.bq), q.device)
        if soft_routing:       # stage-1 router training: gradients flow through the soft mask
            o = sla2_dense(q, k, v, mask, alpha, self.bq, self.bk)
        else:
            a_rows = alpha.repeat_interleave(self.bq, dim=-1)[:, :L]
            o = sparse_linear_attention(q, k, v, lut, self.bq, self.bk, a_rows,
                                        int8=self.use_int8)
        o = o.to(q.dtype)
        if return_sparsity:
            return o, 1.0 - topk / mask.shape[-1]
        return o


class SLA2AttentionImpl(nn.Module):
    """attn_impl with one SLA2 (router + mixing logits) per attention module;
    (b, l, H, hd) duals in and out (reference ``models/sla2_attention.py``)."""

    def __init__(self, head_dim, seq_len, num_heads, topk=0.03, bq=128, bk=64, alpha_init=0.9):
        super().__init__()
        self.seq_len, self.bq, self.bk, self.topk = seq_len, bq, bk, topk
        self.sla2 = SLA2(head_dim, topk=topk, bq=bq, bk=bk, use_int8=False,
                         learnable_router=True, alpha_init=alpha_init)
        init = math.log(alpha_init / (1 - alpha_init))
        self.sla2.alpha_logit = nn.Parameter(torch.full((num_heads, math.ceil(seq_len / bq)), init))

    def forward(self, q, k, v):
        plain = not isinstance(q, Dual)
        q, k, v = (x if isinstance(x, Dual) else Dual(x) for x in (q, k, v))
        fn = lambda a, b, c: self.sla2(a.permute(0, 2, 1, 3), b.permute(0, 2, 1, 3),
                                       c.permute(0, 2, 1, 3)).permute(0, 2, 1, 3).to(a.dtype)
        out = _dual_apply(fn, q, k, v)
        return out.p if plain else out


class SLA2CubeQATAttentionImpl(nn.Module):
    """Cube-tile sparse-linear attention with INT8 QAT (reference
    ``SLA2CubeQATAttentionImpl``): E = prod(tile) tokens per block, routed video
    tiles + always-attended prefix tail blocks, complement over the video tiles.
    Publishes ``logit_max_log2`` (H,) for QK-clip after every training forward."""

    TILE_MAJOR = True

    def __init__(self, head_dim, seq_len, num_heads, grid, tile=(4, 4, 4), topk=0.03,
                 alpha_init=0.9, use_int8=True, pre_permuted=False):
        super().__init__()
        self.pre_permuted = pre_permuted
        self.E = tile[0] * tile[1] * tile[2]
        self.topk_frac, self.use_int8 = topk, use_int8
        n_patch = grid[0] * grid[1] * grid[2]
        self.prefix_len = seq_len - n_patch
        perm, inv, self.Np = tile_permutation(grid, tile, self.prefix_len)
        self.register_buffer("perm", perm, persistent=False)
        self.register_buffer("inv", inv, persistent=False)
        self.n_tail = -(-self.prefix_len // self.E)
        self.Mb = self.Np + self.n_tail
        self.Nb = math.ceil(seq_len / self.E)
        self.register_buffer("a_index", torch.clamp(torch.arange(seq_len) // self.E,
                                                    max=self.Mb - 1), persistent=False)
        self.proj_q = nn.Parameter(torch.eye(head_dim))
        self.proj_k = nn.Parameter(torch.eye(head_dim))
        init = math.log(alpha_init / (1 - alpha_init))
        self.alpha_logit = nn.Parameter(torch.full((num_heads, self.Mb), init))
        self.logit_max_log2: Optional[Tensor] = None

    def route(self, qh: Tensor, kh: Tensor) -> Tuple[Tensor, int]:
        """LUT of routed video tiles plus the prefix tail blocks: (B,H,Mb,T+n_tail)."""
        with torch.no_grad():
            return route_tiles(qh, kh, self.topk_frac, self.Np, self.E, self.prefix_len,
                               self.proj_q, self.proj_k, n_tail=self.n_tail)

    def _core(self, q, k, v, lut_aug):
        """(b, l, H, hd) tile-major -> same, given the routing."""
        qh, kh, vh = (x.permute(0, 2, 1, 3) for x in (q, k, v))
        a_rows = torch.sigmoid(self.alpha_logit)[:, self.a_index]            # (H, L)
        out, _o_s, _o_l, lse = sparse_linear_attention(
            qh, kh, vh, lut_aug, self.E, self.E, a_rows, n_comp_blocks=self.Np,
            int8=self.use_int8, return_parts=True)
        return out.permute(0, 2, 1, 3).to(q.dtype), lse

    def forward(self, q, k, v):
        plain = not isinstance(q, Dual)
        q, k, v = (x if isinstance(x, Dual) else Dual(x) for x in (q, k, v))
        if not self.pre_permuted:
            q, k, v = (x.map(lambda z: z[:, self.perm]) for x in (q, k, v))
        lut_aug, _T = self.route(q.p.detach().permute(0, 2, 1, 3), k.p.detach().permute(0, 2, 1, 3))
        stats = {}

        def fn(a, b, c):
            o, lse = self._core(a, b, c, lut_aug)
            stats["lse"] = lse
            return o
        out = _dual_apply(fn, q, k, v)
        if torch.is_grad_enabled() and (q.p.requires_grad or self.alpha_logit.requires_grad):
            with torch.no_grad():       # per-head max of the sparse-branch LSE, log2 domain
                lse = stats["lse"].detach()
                self.logit_max_log2 = (lse.amax(dim=(0, 2)) * 1.4426950408889634).float()
        if not self.pre_permuted:
            out = out.map(lambda z: z[:, self.inv])
        return out.p if plain else out


def cube_dense_ref(q, k, v, alpha, lut, Np: int, E: int, prefix_len: int):
    """Dense fp32 reference of cube attention (tile-major (B,H,L,D), small L):
    routed video tiles + always-on prefix for the sparse branch; complement =
    non-selected video tiles."""
    B, H, L, D = q.shape
    P = prefix_len
    Mb = lut.shape[2]
    mc = torch.zeros(B, H, Mb, Np, device=q.device).scatter_(-1, lut.long(), 1.0)
    rows = torch.clamp(torch.arange(L, device=q.device) // E, max=Mb - 1)
    m = mc[:, :, rows].repeat_interleave(E, dim=-1)                        # (B,H,L,Np*E)
    if P:
        m = torch.cat([m, torch.ones(B, H, L, P, device=q.device)], -1)
    s = (q.float() @ k.float().transpose(-1, -2)) * D ** -0.5
    o_s = torch.softmax(s.masked_fill(m <= 0, float("-inf")), -1) @ v.float()
    w = F.softmax(q.float(), -1) @ F.softmax(k.float(), -1).transpose(-1, -2)
    comp = 1.0 - m
    if P:
        comp[..., Np * E:] = 0.0
    w = w * comp
    o_l = (w @ v.float()) / (w.sum(-1, keepdim=True) + EPS_LINEAR)
    a = alpha[:, rows].view(1, H, L, 1)
    return a * o_s + (1.0 - a) * o_l


# ------------------------------------------------- CUDA core (fused block) ---
class SparseCore:
    """Attention core for ``ops.block``: block-sparse INT8 tcgen05 kernel for
    the softmax branch (primal + tangent), per-block-state linear branch and
    the alpha mix.  Reverse mode recomputes the op with the torch formulas
    (straight-through for the INT8 grid)."""

    def __init__(self, mod, qblk: int, bk: int, n_comp: Optional[int], int8: bool):
        self.mod, self.qblk, self.bk, self.n_comp, self.int8 = mod, qblk, bk, n_comp, int8

    def _sel_and_alpha(self, qh, kh):
        m = self.mod
        L = qh.shape[2]
        if isinstance(m, SLA2CubeQATAttentionImpl):
            sel, _ = m.route(qh, kh)
            a_rows = torch.sigmoid(m.alpha_logit)[:, m.a_index]
        else:
            with torch.no_grad():
                _, sel, _, _ = m.sla2.router(qh, kh, m.sla2.topk, need_mask=False)
            a_rows = torch.sigmoid(m.sla2.alpha_logit).repeat_interleave(m.bq, dim=-1)[:, :L]
        return sel, a_rows

    def fwd(self, q, k, v, dq, dk, dv, need_bwd: bool):
        from ..ops import sparse as SP

        qh, kh, vh = (x.permute(0, 2, 1, 3) for x in (q, k, v))
        sel, a_rows = self._sel_and_alpha(qh.detach(), kh.detach())
        lut, flags, cnt, fm = SP.route_tables(sel, self.qblk, q.shape[1])
        # inference form (no reverse mode to follow, e.g. the sampler and the guidance passes):
        # no log-sum-exp, no saved state; the same INT8 block-sparse kernel and the same
        # per-key-block states with the alpha mix fused into the apply kernel
        o_s, do_s, lse = SP.sparse_fwd(q, k, v, dq, dk, dv, lut, flags, self.qblk, self.int8,
                                       quant_p=self.int8, need_lse=need_bwd, cnt=cnt)
        flags = fm          # reverse mode needs the (K/V tile, query tile) maps, not the per-tile flags
        from ..ops import linattn as LA

        if LA.AVAILABLE:
            with torch.no_grad():
                o, do, C = LA.forward(q, k, v, dq, dk, dv, o_s, do_s, sel, a_rows, self.qblk,
                                      self.bk, self.n_comp)
                if need_bwd and isinstance(self.mod, SLA2CubeQATAttentionImpl):
                    self.mod.logit_max_log2 = (lse.amax(dim=(0, 2)) * 1.4426950408889634).float()
            return o, do, (sel, lut, flags, o_s, lse, C if need_bwd else None)
        f = lambda a, b, c: linear_branch(a, b, c, sel, self.qblk, self.bk, self.n_comp)
        with torch.no_grad():
            if dq is not None:
                o_l, do_l = torch.func.jvp(f, (qh.float(), kh.float(), vh.float()),
                                           (dq.permute(0, 2, 1, 3).float(),
                                            dk.permute(0, 2, 1, 3).float(),
                                            dv.permute(0, 2, 1, 3).float()))
            else:
                o_l, do_l = f(qh.float(), kh.float(), vh.float()), None
            a = a_rows.detach().t().reshape(1, -1, a_rows.shape[0], 1)       # (1, L, H, 1)
            o = (a * o_s.float() + (1 - a) * o_l.permute(0, 2, 1, 3)).to(q.dtype).contiguous()
            do = None
            if dq is not None:
                do = (a * do_s.float() + (1 - a) * do_l.permute(0, 2, 1, 3)).to(q.dtype).contiguous()
            if need_bwd and isinstance(self.mod, SLA2CubeQATAttentionImpl):
                self.mod.logit_max_log2 = (lse.amax(dim=(0, 2)) * 1.4426950408889634).float()
        return o, do, (sel, lut, flags, o_s, lse, None)

    def bwd(self, q, k, v, o, saved, go, gv_out=None):
        """o = a o_s + (1 - a) o_l: the sparse branch goes through the block-sparse
        backward kernel (S recomputed in bf16 from the fake-quantised operands with the
        forward's LSE: straight-through), the linear branch and alpha through autograd
        of the per-block-state formulas."""
        from ..ops import kernels as K
        from ..ops import sparse as SP

        sel, lut, flags, o_s, lse, C = saved
        m = self.mod
        cube = isinstance(m, SLA2CubeQATAttentionImpl)
        alpha_param = m.alpha_logit if cube else m.sla2.alpha_logit
        B, L, H, D = q.shape
        if C is not None:
            return self._bwd_kernels(q, k, v, saved, go, gv_out, alpha_param, cube)
        with torch.enable_grad():
            a_rows = (torch.sigmoid(alpha_param)[:, m.a_index] if cube else
                      torch.sigmoid(alpha_param).repeat_interleave(m.bq, dim=-1)[:, :L])
            ql, kl, vl = (x.detach().permute(0, 2, 1, 3).float().requires_grad_(True)
                          for x in (q, k, v))
            o_l = linear_branch(ql, kl, vl, sel, self.qblk, self.bk, self.n_comp)
            a = a_rows.t().reshape(1, L, H, 1)
            gof = go.float()
            mix = (a * o_s.float().detach() + (1 - a) * o_l.permute(0, 2, 1, 3))
            gq_l, gk_l, gv_l, ga = torch.autograd.grad(mix, (ql, kl, vl, alpha_param), gof)
        alpha_param.grad = ga if alpha_param.grad is None else alpha_param.grad + ga
        with torch.no_grad():
            g_os = (a.detach() * gof).to(q.dtype).contiguous()
            qq, kk, vv = q, k, v
            if self.int8:
                _, _, qq = SP.quantize_blocks(K._tma_ok(q), self.qblk, want_q=False, want_fq=True)
                _, _, kk = SP.quantize_blocks(K._tma_ok(k), 64, want_q=False, want_fq=True)
                _, _, vv = SP.quantize_blocks(K._tma_ok(v), 64, want_q=False, want_fq=True)
            qlist, qflags, qrank = SP.kv_lists(flags, want_rank=True)   # `flags`: the maps (see fwd)
            gq_s, gk_s, gv_s = K.attn_bwd(qq, kk, vv, o_s, lse, g_os, qlist=qlist, qflags=qflags,
                                          qrank=qrank)
            back = lambda t: t.permute(0, 2, 1, 3)
            gq = (gq_s.float() + back(gq_l)).to(q.dtype)
            gk = (gk_s.float() + back(gk_l)).to(q.dtype)
            gv = (gv_s.float() + back(gv_l)).to(q.dtype)
            if gv_out is not None:
                gv_out.copy_(gv)
                gv = gv_out
        return gq, gk, gv


def _sparse_core_bwd_kernels(self, q, k, v, saved, go, gv_out, alpha_param, cube):
    """Reverse mode with the linear branch on this library's kernels: row side first
    (it produces the sparse branch's upstream gradient a*go), then the block-sparse
    backward kernel, then the key side, which adds both branches."""
    from ..ops import kernels as K
    from ..ops import linattn as LA
    from ..ops import sparse as SP

    sel, lut, flags, o_s, lse, C = saved
    m = self.mod
    B, L, H, D = q.shape
    with torch.no_grad():
        a_rows = (torch.sigmoid(alpha_param)[:, m.a_index] if cube else
                  torch.sigmoid(alpha_param).repeat_interleave(m.bq, dim=-1)[:, :L])
        gq_l, gnum, gden, ga_row, g_os = LA.backward_rows(q, o_s, go, C, a_rows, self.qblk)
        Mb = -(-L // self.qblk)
        ga = F.pad(ga_row.sum(0), (0, Mb * self.qblk - L)).view(H, Mb, self.qblk).sum(-1)
        if ga.shape[1] < alpha_param.shape[1]:
            ga = F.pad(ga, (0, alpha_param.shape[1] - ga.shape[1]))
        ga = ga.to(alpha_param.dtype)
        alpha_param.grad = ga if alpha_param.grad is None else alpha_param.grad + ga
        qq, kk, vv = q, k, v
        if self.int8 and self.qblk == 64:
            (_, _, qq), (_, _, kk), (_, _, vv) = SP.quantize_blocks_many(
                [(q, False, True), (k, False, True), (v, False, True)])
        elif self.int8:
            _, _, qq = SP.quantize_blocks(K._tma_ok(q), self.qblk, want_q=False, want_fq=True)
            _, _, kk = SP.quantize_blocks(K._tma_ok(k), 64, want_q=False, want_fq=True)
            _, _, vv = SP.quantize_blocks(K._tma_ok(v), 64, want_q=False, want_fq=True)
        qlist, qflags, qrank = SP.kv_lists(flags, want_rank=True)       # `flags`: the maps (see fwd)
        # the linear branch's query gradient rides into the block-sparse backward's dQ epilogue
        gq, gk_s, gv_s = K.attn_bwd(qq, kk, vv, o_s, lse, g_os, qlist=qlist, qflags=qflags,
                                    qrank=qrank, dq_add=gq_l)
        gk, gv = LA.backward_kv(q, k, v, gnum, gden, sel, gk_s, gv_s, self.qblk, self.bk,
                                self.n_comp, gv_out=gv_out)
    return gq, gk, gv


SparseCore._bwd_kernels = _sparse_core_bwd_kernels


def _cuda_sparse_ready(t: Tensor) -> bool:
    if not t.is_cuda:
        return False
    from ..ops import cuda as cu

    if not cu.available():
        return False
    from ..ops import kernels as K

    return K._has("imf_attn_sparse_fwd")


def _cube_fused_core(self):
    if self.E != 64 or not _cuda_sparse_ready(self.alpha_logit) or not self.pre_permuted:
        return None
    return SparseCore(self, 64, 64, self.Np, self.use_int8)


def _sla2_fused_core(self):
    if self.bk != 64 or self.bq not in (64, 128) or not _cuda_sparse_ready(self.sla2.alpha_logit):
        return None
    return SparseCore(self, self.bq, 64, None, False)


SLA2CubeQATAttentionImpl.fused_core = property(_cube_fused_core)
SLA2AttentionImpl.fused_core = property(_sla2_fused_core)
