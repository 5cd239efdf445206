"""One MLA transformer block as a single autograd node on the sm_100a kernels.

Forward evaluates primal and tangent together (tangent rows sit right behind
the primal rows, so every GEMM is one launch over 2*b*l rows); backward is the
hand-scheduled reverse pass through the primal only.  Per block the forward is
11 fused launches + attention, instead of ~120 framework kernels; this is the
production path on CUDA, the generic ``ops.dual`` composition stays as the CPU
path and oracle.

Block structure (reference ``models/imf_dit_video.py:909-972``, ``:422-467``):
    n1  = norm1(remix(prefix, snaps; w1))
    a_  = n1 [q_a | kv_a | g]^T ; latent norms ; q_b, kv_b ; q/k prep
    o   = attention(q, k, v) * sigmoid(g) ; a = o out^T
    p2  = (fresh ? 0 : prefix) + a * attn_scale ; snaps2 = snaps (+ prefix if fresh)
    n2  = norm2(remix(p2, snaps2; w2))
    m   = situ(n2 [w1 | w3]^T) w2^T ;  out = p2 + m * mlp_scale
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import kernels as K
from . import rowops as R

BF16, F32 = torch.bfloat16, torch.float32


class DenseCore:
    """Dense softmax attention core: fused primal+tangent forward kernel and
    reverse-mode kernel.  SLA2 cores implement the same two methods."""

    def fwd(self, q, k, v, dq, dk, dv, need_bwd: bool):
        o, do, lse = K.attn_fwd(q, k, v, dq, dk, dv, need_lse=need_bwd)
        return o, do, (lse,)

    def bwd(self, q, k, v, o, saved, go, gv_out: Optional[torch.Tensor] = None):
        (lse,) = saved
        if K._has("imf_attn_bwd"):
            return K.attn_bwd(q, k, v, o, lse, go, gv_out=gv_out)
        gq, gk, gv = K._sdpa_backward(q, k, v, go)
        if gv_out is not None:
            gv_out.copy_(gv)
            gv = gv_out
        return gq, gk, gv


DENSE_CORE = DenseCore()


class GradSinks:
    """Where the weight gradients of one block go.  The six bf16 matrices the node works on
    are casts / concatenations of fp32 parameters; ``pieces[name]`` lists, for matrix
    ``name``, the parameters it was built from as (param, first_row, n_rows, n_cols).

    When every such parameter already owns an fp32 ``.grad`` buffer (the flat gradient
    arena of the optimizer engine, or a previous micro-batch's gradient), the backward
    pass writes each product dY^T X straight into it with accumulation and returns no
    gradient for the matrices: no bf16 gradient tensors, no casts, no splits, no adds."""

    ORDER = ("W_a", "W_qb", "W_kvb", "W_out", "W13", "W2")
    SMALL = ("g_n1", "g_n2", "g_qa", "g_kva", "g_qn", "g_kn", "a_scale", "m_scale")

    def __init__(self, pieces, small=None):
        self.pieces = pieces
        self.small = small or {}      # the 1-D parameters (gains, gates) by their role
        self.on_backward = None       # optional callable: this block's backward has begun
        self.mats_cached = False      # the last forward used weight copies without autograd history

    def small_dst(self, name: str):
        """fp32 gradient buffer of the 1-D parameter in role ``name`` (flattened), or None."""
        p = self.small.get(name)
        if p is None or p.grad is None or p.grad.dtype != F32 or not p.grad.is_contiguous():
            return None
        return p.grad.view(-1)

    def direct(self) -> bool:
        if any(self.small_dst(nm) is None for nm in self.SMALL):
            return False
        for name in self.ORDER:
            for p, r0, _n, _c in self.pieces[name]:
                g = p.grad
                if (not p.requires_grad or g is None or g.dtype != F32 or not g.is_contiguous()
                        or g.shape != p.shape or r0 % 8 or g.data_ptr() % 16):
                    return False       # r0: the TMA view of dY[:, r0:] must start 16-byte aligned
        return True

    def accumulate(self, name: str, dy: torch.Tensor, x: torch.Tensor) -> None:
        """grad(piece) += dy[:, rows of the piece]^T x[:, :cols of the piece]"""
        for p, r0, n, c in self.pieces[name]:
            K.gemm_wgrad(dy[:, r0:r0 + n], x[:, :c] if c != x.shape[1] else x,
                         out=p.grad.view(n, c), accumulate=True)


class BlockGeom:
    """Static geometry of a block (python ints only)."""

    def __init__(self, attn, hidden: int, fpad: int):
        self.d = hidden
        self.H = attn.num_heads
        self.dq, self.dc = attn.q_lora_rank, attn.kv_lora_rank
        self.dn, self.dr, self.dv = attn.qk_nope_head_dim, attn.qk_rope_head_dim, attn.v_head_dim
        self.hd = self.dn + self.dr
        self.gate = attn.use_output_gate
        self.na = self.dq + self.dc + self.dr + (self.H * self.dv if self.gate else 0)
        self.fp = fpad


def supported(g: BlockGeom) -> bool:
    return (g.d % 128 == 0 and g.hd in (64, 128) and g.dv == g.hd and g.dq % 8 == 0 and g.dc % 8 == 0
            and g.dr % 2 == 0 and g.dn % (g.hd // 32) == 0 and (g.H * g.dv) % 8 == 0
            and (g.dq + g.dc) % 4 == 0 and g.fp % 8 == 0)


class _BlockFn(torch.autograd.Function):
    """inputs: geom, core, flags, eps, beta, lbeta, cos, sin, nsnap,
    prefix, dprefix, *snaps, *dsnaps,
    w1, w2, g_norm1, g_norm2, g_qa, g_kva, g_qn, g_kn, attn_scale, mlp_scale,
    W_a, W_qb, W_kvb, W_out, W13, W2
    outputs: new_prefix (fp32), new_dprefix (fp32 or empty)."""

    @staticmethod
    def forward(ctx, geom, core, fresh, use_res, eps, beta, lbeta, cos, sin, nsnap, prefix,
                dprefix, *rest):
        g: BlockGeom = geom
        core, sinks = core if isinstance(core, tuple) else (core, None)
        snaps = list(rest[:nsnap])
        dsnaps = list(rest[nsnap:2 * nsnap])
        (w1, w2, g_n1, g_n2, g_qa, g_kva, g_qn, g_kn, a_scale, m_scale,
         W_a, W_qb, W_kvb, W_out, W13, W2) = rest[2 * nsnap:]
        has_t = dprefix is not None
        need_bwd = any(ctx.needs_input_grad)
        B, L, d = prefix.shape
        rows = B * L
        dev = prefix.device
        T = 2 if has_t else 1
        flat = lambda t: None if t is None else t.reshape(rows, d)
        pfx, dpfx = flat(prefix), flat(dprefix)
        sn = [flat(s) for s in snaps]
        dsn = [flat(s) if has_t else None for s in dsnaps] if has_t else [None] * nsnap
        new = lambda *shape, dt=BF16: torch.empty(*shape, dtype=dt, device=dev)

        # 1. remix + norm1
        n1 = new(T, rows, d)
        R.resnorm_fwd(pfx, dpfx, None, None, None, sn, dsn, w1 if (use_res and nsnap) else None,
                      g_n1, eps, n1[0], n1[1] if has_t else None, None, None)
        # 2. fused projection GEMM over primal+tangent rows
        a_ = K.gemm(n1.view(T * rows, d), W_a)                       # [T*rows, na]
        na = g.na
        # 3. latent norms
        qlat, kvlat = new(T, rows, g.dq), new(T, rows, g.dc)
        a0, a1 = a_[:rows], (a_[rows:] if has_t else None)
        R.rmsnorm_seg_fwd(
            [(a0, a1, g_qa, qlat[0], qlat[1] if has_t else None, g.dq, na, g.dq),
             (a0[:, g.dq:], None if a1 is None else a1[:, g.dq:], g_kva, kvlat[0],
              kvlat[1] if has_t else None, g.dc, na, g.dc)], rows, eps, has_t)
        # 4. up-projections
        qb = K.gemm(qlat.view(T * rows, g.dq), W_qb)                 # [T*rows, H*hd]
        kvb = K.gemm(kvlat.view(T * rows, g.dc), W_kvb)              # [T*rows, H*(dn+dv)]
        # 5. q / k preparation
        q, k = new(T, B, L, g.H, g.hd), new(T, B, L, g.H, g.hd)
        kr0 = a0[:, g.dq + g.dc:]
        kr1 = None if a1 is None else a1[:, g.dq + g.dc:]
        R.qkprep_fwd(qb[:rows], qb[rows:] if has_t else None, kvb[:rows],
                     kvb[rows:] if has_t else None, kr0, kr1, cos, sin, g_qn, g_kn,
                     q[0], q[1] if has_t else None, k[0], k[1] if has_t else None,
                     rows, L, g.H, g.dn, g.dr, g.dv, na, eps)
        kv4 = kvb.view(T, B, L, g.H, g.dn + g.dv)
        v0 = kv4[0][..., g.dn:]
        v1 = kv4[1][..., g.dn:] if has_t else None
        # 6. attention core
        o, do, core_saved = core.fwd(q[0], k[0], v0, q[1] if has_t else None,
                                     k[1] if has_t else None, v1, need_bwd)
        hv = g.H * g.dv
        # 7. output gate
        if g.gate:
            og = new(T, rows, hv)
            gcol = g.dq + g.dc + g.dr
            R.outgate_fwd(o.view(rows, hv), None if do is None else do.view(rows, hv),
                          a0[:, gcol:], None if a1 is None else a1[:, gcol:], og[0],
                          og[1] if has_t else None, rows, hv, hv, na)
        else:
            og = torch.stack([o.view(rows, hv), do.view(rows, hv)]) if has_t else o.view(1, rows, hv)
        # 8. output projection
        a_out = K.gemm(og.view(T * rows, hv), W_out)                 # [T*rows, d]
        # 9. residual + remix + norm2
        p2, n2 = new(T, rows, d, dt=F32), new(T, rows, d)
        sn2 = sn + [pfx] if fresh else sn
        dsn2 = (dsn + [dpfx]) if fresh else dsn
        R.resnorm_fwd(None if fresh else pfx, None if fresh else dpfx, a_out[:rows],
                      a_out[rows:] if has_t else None, a_scale, sn2, dsn2,
                      w2 if use_res else None, g_n2, eps, n2[0], n2[1] if has_t else None,
                      p2[0], p2[1] if has_t else None)
        # 10. MLP
        gu = K.gemm(n2.view(T * rows, d), W13)                       # [T*rows, 2*fp]
        act = new(T * rows, g.fp)
        R.situ_fwd(gu[:rows], gu[rows:] if has_t else None, act[:rows],
                   act[rows:] if has_t else None, rows, g.fp, beta, lbeta)
        m = K.gemm(act, W2)                                          # [T*rows, d]
        # 11. residual
        out = new(T, rows, d, dt=F32)
        R.scale_add_fwd(p2[0], p2[1] if has_t else None, m[:rows], m[rows:] if has_t else None,
                        m_scale, out[0], out[1] if has_t else None, rows, d)
        if need_bwd:
            ctx.save_for_backward(prefix, *snaps, w1, w2, g_n1, g_n2, g_qa, g_kva, g_qn, g_kn,
                                  a_scale, m_scale, W_a, W_qb, W_kvb, W_out, W13, W2, cos, sin,
                                  n1[0], a_[:rows], qlat[0], kvlat[0], qb[:rows], kvb[:rows],
                                  q[0], k[0], o, og[0], a_out[:rows], p2[0], n2[0], gu[:rows],
                                  act[:rows], m[:rows], *core_saved)
            ctx.meta = (g, core, fresh, use_res, eps, beta, lbeta, nsnap, B, L, len(core_saved))
            ctx.sinks = sinks
            ctx.mats_cached = bool(getattr(sinks, "mats_cached", False))
        new_p = out[0].view(B, L, d)
        new_t = out[1].view(B, L, d) if has_t else out.new_empty(0)
        ctx.mark_non_differentiable(new_t)
        return new_p, new_t

    @staticmethod
    def backward(ctx, g_out, _g_t):
        g, core, fresh, use_res, eps, beta, lbeta, nsnap, B, L, ncore = ctx.meta
        sv = ctx.saved_tensors
        prefix = sv[0]
        snaps = list(sv[1:1 + nsnap])
        (w1, w2, g_n1, g_n2, g_qa, g_kva, g_qn, g_kn, a_scale, m_scale, W_a, W_qb, W_kvb, W_out,
         W13, W2, cos, sin, n1, a_, qlat, kvlat, qb, kvb, q, k, o, og, a_out, p2, n2, gu, act,
         m) = sv[1 + nsnap:1 + nsnap + 34]
        core_saved = sv[1 + nsnap + 34:]
        rows, d = B * L, g.d
        dev = prefix.device
        hv, na = g.H * g.dv, g.na
        pfx = prefix.reshape(rows, d)
        sn = [s.reshape(rows, d) for s in snaps]
        g_out = g_out.reshape(rows, d).contiguous()
        new = lambda *shape, dt=BF16: torch.empty(*shape, dtype=dt, device=dev)
        if getattr(ctx, "sinks", None) is not None and ctx.sinks.on_backward is not None:
            ctx.sinks.on_backward()

        # data gradients dY W: W is [n_out, n_in] = [K, N], consumed MN-major as it is.
        # weight gradients dY^T X: split-K products (K = token rows), written straight into the
        # parameters' gradient buffers when they exist (`direct`), else returned to autograd.
        # The gains' / gates' gradients come out of the row kernels as per-CTA partial sums; one
        # launch at the end adds them all up, into the same kind of destination.
        sinks = getattr(ctx, "sinks", None)
        direct = sinks is not None and sinks.direct()
        if not direct and getattr(ctx, "mats_cached", False):
            # the forward used cached weight copies without autograd history because the
            # gradient buffers existed then; returned gradients would reach no parameter
            raise RuntimeError("the parameters' fp32 gradient buffers were removed between the "
                               "forward and the backward pass of a fused block")
        wgrad = (lambda name, dy, x: sinks.accumulate(name, dy, x)) if direct else \
            (lambda name, dy, x: K.gemm_wgrad(dy, x).to(BF16))
        cs = R.ColSums()
        small = (lambda name, part, col, D: (cs.add(part, col, D, sinks.small_dst(name)), None)[1]) \
            if direct else (lambda name, part, col, D: cs.add(part, col, D, None))

        # 11'. out = p2 + m * mlp_scale
        g_m, part_ms = R.scale_add_bwd(m, m_scale, g_out, rows, d, raw=True)
        g_mscale = small("m_scale", part_ms, 0, d)
        # 10'. MLP
        g_act = K.gemm(g_m, W2, b_mn=True)                          # [rows, fp]
        gW2 = wgrad("W2", g_m, act)
        g_gu = new(rows, 2 * g.fp)
        R.situ_bwd(gu, g_act, g_gu, rows, g.fp, beta, lbeta)
        g_n2v = K.gemm(g_gu, W13, b_mn=True)
        gW13 = wgrad("W13", g_gu, n2)
        # 9'. residual + remix + norm2
        sn2 = sn + [pfx] if fresh else sn
        g_res2, g_aout, g_sn2, part2 = R.resnorm_bwd(
            None if fresh else pfx, a_out, a_scale, sn2, w2 if use_res else None, g_n2, eps,
            g_n2v, g_out, want_g_res=not fresh, raw=True)
        gg_n2 = small("g_n2", part2, 0, d)
        g_w2 = cs.add(part2, 1, d, None) if use_res else None       # product of two parameters
        g_ascale = small("a_scale", part2, 2, d)
        # 8'. output projection
        g_og = K.gemm(g_aout, W_out, b_mn=True)                     # [rows, hv]
        gW_out = wgrad("W_out", g_aout, og)
        # 7'. output gate (gate gradient goes straight into its band of g_a_)
        g_a = new(rows, na)
        o2 = o.view(rows, hv)
        if g.gate:
            gcol = g.dq + g.dc + g.dr
            g_o = new(rows, hv)
            R.outgate_bwd(o2, a_[:, gcol:], g_og, g_o, g_a[:, gcol:], rows, hv, hv, na, hv, na)
        else:
            g_o = g_og
        # 6'. attention (value gradient goes straight into its band of g_kvb)
        g_kvb = new(rows, g.H * (g.dn + g.dv))
        kv4 = kvb.view(B, L, g.H, g.dn + g.dv)
        gkv4 = g_kvb.view(B, L, g.H, g.dn + g.dv)
        gq, gk, _gv = core.bwd(q, k, kv4[..., g.dn:], o, core_saved, g_o.view(B, L, g.H, g.dv),
                               gv_out=gkv4[..., g.dn:])
        # 5'. q / k preparation
        g_qb = new(rows, g.H * g.hd)
        part_qk = R.qkprep_bwd(qb, kvb, cos, sin, g_qn, g_kn, gq.contiguous(),
                                gk.contiguous(), g_qb, g_kvb, g_a[:, g.dq + g.dc:], rows, L,
                                g.H, g.dn, g.dr, g.dv, na, eps, raw=True)
        gg_qn = small("g_qn", part_qk, 0, g.dn)
        gg_kn = small("g_kn", part_qk, 1, g.dn)
        # 4'. up-projections
        g_qlat = K.gemm(g_qb, W_qb, b_mn=True)
        gW_qb = wgrad("W_qb", g_qb, qlat)
        g_kvlat = K.gemm(g_kvb, W_kvb, b_mn=True)
        gW_kvb = wgrad("W_kvb", g_kvb, kvlat)
        # 3'. latent norms (write into the q / kv bands of g_a_)
        part_qa, part_kva = R.rmsnorm_seg_bwd(
            [(a_, g_qa, g_qlat, g_a, g.dq, na, g.dq),
             (a_[:, g.dq:], g_kva, g_kvlat, g_a[:, g.dq:], g.dc, na, g.dc)], rows, eps, raw=True)
        gg_qa = small("g_qa", part_qa, 0, g.dq)
        gg_kva = small("g_kva", part_kva, 0, g.dc)
        # 2'. fused projection
        g_n1v = K.gemm(g_a, W_a, b_mn=True)
        gW_a = wgrad("W_a", g_a, n1)
        # 1'. remix + norm1; the prefix gradient of step 9' rides in as g_pfx_ext
        ext = g_sn2[-1] if fresh else g_res2
        # the snapshot gradients of step 9' are added in by the kernel (no separate adds)
        g_pfx, _, g_sn1, part1 = R.resnorm_bwd(
            pfx, None, None, sn, w1 if (use_res and nsnap) else None, g_n1, eps, g_n1v, ext,
            raw=True, g_snaps_ext=g_sn2[:nsnap] if (use_res and nsnap) else None)
        gg_n1 = small("g_n1", part1, 0, d)
        g_w1 = cs.add(part1, 1, d, None) if (use_res and nsnap) else None
        cs.flush()
        g_snaps = []
        for j in range(nsnap):
            g_snaps.append((g_sn1[j] if (use_res and nsnap) else g_sn1[j].add_(g_sn2[j]))
                           .view(B, L, d))
        if g_w1 is None:
            g_w1 = torch.zeros_like(w1) if w1 is not None else None
        if g_w2 is None:
            g_w2 = torch.zeros_like(w2) if w2 is not None else None
        grads = (None,) * 10 + (g_pfx.view(B, L, d), None) + tuple(g_snaps) + (None,) * nsnap + (
            g_w1, g_w2, gg_n1, gg_n2, gg_qa, gg_kva, gg_qn, gg_kn, g_ascale, g_mscale,
            gW_a, gW_qb, gW_kvb, gW_out, gW13, gW2)
        return grads


def run_block(geom: BlockGeom, core, fresh: bool, use_res: bool, eps: float, beta: float,
              lbeta: Optional[float], cos, sin, prefix, dprefix, snaps, dsnaps, params,
              sinks: Optional[GradSinks] = None):
    """params: (w1, w2, g_norm1, g_norm2, g_qa, g_kva, g_qn, g_kn, attn_scale, mlp_scale,
    W_a, W_qb, W_kvb, W_out, W13, W2) with bf16 weight matrices; ``sinks`` says which
    parameters those matrices were built from (see ``GradSinks``)."""
    nsnap = len(snaps)
    if sinks is not None:
        core = (core, sinks)
    args = list(snaps) + ([s for s in dsnaps] if dprefix is not None else [None] * nsnap)
    p, t = _BlockFn.apply(geom, core, fresh, use_res, eps, beta, lbeta, cos, sin, nsnap, prefix,
                          dprefix, *args, *params)
    return p, (t if dprefix is not None else None)


class _OutHeadFn(torch.autograd.Function):
    """Output attention-residual re-mix + the final layer's RMSNorm as one kernel:
        n = RMSNorm(remix(prefix, snaps; w)) * gain            (bf16, + tangent)
    inputs: eps, nsnap, prefix, dprefix, *snaps, *dsnaps, w, gain.  The tangent is not
    differentiated.  (reference models/imf_dit_video.py:287-320, :535-549)"""

    @staticmethod
    def forward(ctx, eps, nsnap, prefix, dprefix, *rest):
        snaps, dsnaps = list(rest[:nsnap]), list(rest[nsnap:2 * nsnap])
        w, gain = rest[2 * nsnap:]
        B, L, d = prefix.shape
        rows = B * L
        has_t = dprefix is not None
        flat = lambda t: None if t is None else t.reshape(rows, d)
        n = torch.empty(rows, d, dtype=BF16, device=prefix.device)
        dn = torch.empty_like(n) if has_t else None
        R.resnorm_fwd(flat(prefix), flat(dprefix), None, None, None, [flat(s) for s in snaps],
                      [flat(s) if has_t else None for s in dsnaps] if has_t else [None] * nsnap,
                      w, gain, eps, n, dn, None, None)
        K.LAUNCHES.count += 1
        ctx.save_for_backward(prefix, w, gain, *snaps)
        ctx.meta = (eps, nsnap, B, L, d)
        ctx.set_materialize_grads(False)
        return n.view(B, L, d), (dn.view(B, L, d) if has_t else None)

    @staticmethod
    def backward(ctx, gn, _gdn):
        eps, nsnap, B, L, d = ctx.meta
        prefix, w, gain, *snaps = ctx.saved_tensors
        rows = B * L
        g_res, _, g_sn, g_gain, g_w, _ = R.resnorm_bwd(
            prefix.reshape(rows, d), None, None, [s.reshape(rows, d) for s in snaps], w, gain,
            eps, gn.reshape(rows, d).contiguous(), None)
        K.LAUNCHES.count += 1
        grads = (None, None, g_res.view(B, L, d), None) + tuple(g.view(B, L, d) for g in g_sn) + \
            (None,) * nsnap + (g_w, g_gain)
        return grads


def out_head(prefix, snaps, w: torch.Tensor, gain: torch.Tensor, eps: float):
    """``prefix`` / ``snaps``: Dual (fp32 (B, L, d)); returns (n, dn) bf16."""
    ns = len(snaps)
    has_t = prefix.t is not None
    dsn = [(s.t if s.t is not None else torch.zeros_like(s.p)) for s in snaps] if has_t else [None] * ns
    return _OutHeadFn.apply(float(eps), ns, prefix.p.contiguous(),
                            prefix.t.contiguous() if has_t else None,
                            *[s.p.contiguous() for s in snaps], *dsn,
                            w.float().contiguous(), gain.float().contiguous())
