"""iMF video DiT (MLA attention, in-context conditioning, gated residuals,
attention-residual heads, u/v output branches) evaluated on dual numbers.

Capabilities, module names and parameter shapes follow the reference model
(``models/imf_dit_video.py:610-1070``) so that ``state_dict()`` keys are
identical and reference checkpoints load unchanged.  The evaluation strategy
is different: the forward runs on ``ops.dual.Dual`` values, so ONE pass gives
the primal (with its autograd graph), the d/dt tangent of the u branch, and
the v branch; the guidance passes can skip the u branch entirely.

Numerics policy on CUDA: fp32 master parameters, fp32 residual stream,
``compute_dtype`` (bf16) for every GEMM operand, q/k/v and attention output.
"""

from __future__ import annotations

import math
from functools import partial
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..ops import dual as D
from ..ops.dual import Dual
from ..ops.patch import permute_rows

Tensor = torch.Tensor


# ------------------------------------------------------------------ init ---
def scaled_variance_linear(fan_in: int, fan_out: int, bias: bool, init_constant: float
                           ) -> nn.Linear:
    """weight ~ N(0, (init_constant / sqrt(fan_in))^2), zero bias
    (reference ``models/imf_dit_video.py:112-118``)."""
    lin = nn.Linear(fan_in, fan_out, bias=bias)
    with torch.no_grad():
        lin.weight.normal_(0.0, init_constant / math.sqrt(fan_in))
        if bias:
            lin.bias.zero_()
    return lin


# --------------------------------------------------------------- modules ---
class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x, out_dtype=None):
        if isinstance(x, Dual):
            return D.rmsnorm(x, self.weight, self.eps, out_dtype)
        return D.rmsnorm(Dual(x), self.weight, self.eps, out_dtype).p


class SituAndMul(nn.Module):
    """beta tanh(g/beta) sigmoid(g) * linear_beta tanh(up/linear_beta)
    (reference ``models/imf_dit_video.py:136-165``)."""

    def __init__(self, beta: float = 1.0, linear_beta: Optional[float] = None):
        super().__init__()
        self.beta, self.linear_beta = beta, linear_beta

    def forward(self, gate: Dual, up: Dual) -> Dual:
        return D.situ_mul(D.lift(gate), D.lift(up), self.beta, self.linear_beta)


class SwiGLUMlp(nn.Module):
    def __init__(self, dim: int, hidden: int, weight_init_constant: float = 1.0,
                 situ_beta: float = 1.0, situ_linear_beta: Optional[float] = None):
        super().__init__()
        mk = partial(scaled_variance_linear, bias=False, init_constant=weight_init_constant)
        self.w1 = mk(dim, hidden)      # gate
        self.w3 = mk(dim, hidden)      # up
        self.w2 = mk(hidden, dim)      # down
        self.act = SituAndMul(situ_beta, situ_linear_beta)

    def forward(self, x: Dual) -> Dual:
        x = D.lift(x)
        f = self.w1.out_features
        w1, w3, w2 = self.w1.weight, self.w3.weight, self.w2.weight
        # TMA-fed GEMMs need row strides that are multiples of 16 bytes: pad the
        # hidden width with zero rows/columns (exact: situ(0, 0) = 0)
        pad = (-f) % 8 if x.p.is_cuda else 0
        if pad:
            z = w1.new_zeros(pad, w1.shape[1])
            w13 = torch.cat([w1, z, w3, z], dim=0)
            w2 = torch.nn.functional.pad(w2, (0, pad))
        else:
            w13 = torch.cat([w1, w3], dim=0)
        fp = f + pad
        gu = D.linear(x, w13)                      # one GEMM for [gate | up]
        gate = gu.map(lambda z_: z_[..., :fp])
        up = gu.map(lambda z_: z_[..., fp:])
        return D.linear(self.act(gate, up), w2)


def sinusoid(t: Tensor, dim: int, max_period: float = 10000.0) -> Tuple[Tensor, Tensor]:
    """cos|sin features of a scalar and their derivative w.r.t. the scalar."""
    if t.is_cuda and not t.requires_grad and t.dim() == 1:
        from ..ops import patch as PK

        if PK.AVAILABLE and not torch._C._are_functorch_transforms_active():
            return PK.sinusoid(t, dim, max_period)
    half = dim // 2
    freqs = torch.exp(-math.log(max_period)
                      * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    arg = t[:, None].float() * freqs[None]
    c, s = torch.cos(arg), torch.sin(arg)
    emb = torch.cat([c, s], dim=-1)
    demb = torch.cat([-s * freqs[None], c * freqs[None]], dim=-1)
    if dim % 2:
        z = torch.zeros_like(emb[:, :1])
        emb, demb = torch.cat([emb, z], -1), torch.cat([demb, z], -1)
    return emb, demb


class TimestepEmbedder(nn.Module):
    """sinusoid(freq) -> Linear -> SiLU -> Linear."""

    def __init__(self, hidden_size: int, frequency_embedding_size: int = 256,
                 init_constant: float = 1.0):
        super().__init__()
        self.frequency_embedding_size = frequency_embedding_size
        mk = partial(scaled_variance_linear, bias=True, init_constant=init_constant)
        self.mlp = nn.Sequential(mk(frequency_embedding_size, hidden_size), nn.SiLU(),
                                 mk(hidden_size, hidden_size))

    @staticmethod
    def timestep_embedding(t: Tensor, dim: int, max_period: float = 10000.0) -> Tensor:
        return sinusoid(t, dim, max_period)[0]

    def forward(self, t) -> Dual:
        t = D.lift(t)
        emb, demb = sinusoid(t.p, self.frequency_embedding_size)
        l0, l2 = self.mlp[0], self.mlp[2]
        dt = l0.weight.dtype
        x = Dual(emb.to(dt), None if t.t is None else (demb * t.t[:, None].float()).to(dt))
        h = D.linear(x, l0.weight, l0.bias)
        sg = torch.sigmoid(h.p)
        a = Dual(h.p * sg, None if h.t is None
                 else h.t * (sg * (1 + h.p * (1 - sg))).detach())
        return D.linear(a, l2.weight, l2.bias)


class LabelEmbedder(nn.Module):
    def __init__(self, num_classes: int, hidden_size: int, init_constant: float = 1.0):
        super().__init__()
        self.embedding_table = nn.Embedding(num_classes + 1, hidden_size)
        with torch.no_grad():
            self.embedding_table.weight.normal_(0.0, init_constant / math.sqrt(hidden_size))

    def forward(self, labels: Tensor) -> Tensor:
        return self.embedding_table(labels)


class VideoPatchEmbedder(nn.Module):
    """Conv3d(kernel = stride = patch) stored as a conv (checkpoint parity),
    evaluated as patch-gather + GEMM so the tangent is one more row block."""

    def __init__(self, in_channels: int, hidden_size: int, patch_size=(1, 2, 2),
                 bias: bool = True):
        super().__init__()
        self.patch_size = tuple(patch_size)
        self.proj = nn.Conv3d(in_channels, hidden_size, kernel_size=self.patch_size,
                              stride=self.patch_size, bias=bias)
        with torch.no_grad():
            nn.init.xavier_uniform_(self.proj.weight.view(hidden_size, -1))
            if bias:
                self.proj.bias.zero_()

    def patches(self, x: Tensor) -> Tensor:
        """(b, c, t, h, w) -> (b, gt*gh*gw, c*pt*ph*pw): one gather kernel on CUDA."""
        from ..ops.patch import patch_rows

        return patch_rows(x, self.patch_size, c_last=False)

    def forward(self, x) -> Dual:
        x = D.lift(x).map(self.patches)
        w = self.proj.weight.reshape(self.proj.weight.shape[0], -1)
        return D.linear(x, w, self.proj.bias)


# ------------------------------------------------- attention plug-ins -----
def _plug(q, k, v, impl: str):
    """Plug-ins take duals inside the model; called with plain (b, l, H, d) tensors (the
    reference's ``attn_impl(q, k, v)`` protocol) they return a plain tensor."""
    plain = not isinstance(q, Dual)
    out = D.dense_attention(D.lift(q), D.lift(k), D.lift(v), impl=impl)
    return out.p if plain else out


def flash_jvp_attention(q, k, v):
    """Fused primal+tangent dense attention (sm_100a kernel on CUDA)."""
    return _plug(q, k, v, "auto")


def sdpa_math_attention(q, k, v):
    return _plug(q, k, v, "math")


def sdpa_flash_attention(q, k, v):
    return _plug(q, k, v, "sdpa")


eager_math_attention = sdpa_math_attention


def _is_factory(impl) -> bool:
    return isinstance(impl, type) or (isinstance(impl, partial) and isinstance(impl.func, type))


class MLAAttention(nn.Module):
    """Multi-head latent attention with decoupled partial RoPE
    (reference ``models/imf_dit_video.py:323-467``): q: d->dq->norm->H(dn+dr);
    kv: d->(dc | dr shared rotary key); dc->norm->H(dn+dv); per-head RMSNorm on
    the nope bands; sigmoid output gate; no biases."""

    def __init__(self, hidden_size, num_heads, q_lora_rank, kv_lora_rank,
                 qk_nope_head_dim, qk_rope_head_dim, v_head_dim,
                 weight_init_constant=1.0, norm_eps=1e-6,
                 attn_impl: Callable = sdpa_math_attention, use_output_gate=True):
        super().__init__()
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.q_lora_rank, self.kv_lora_rank = q_lora_rank, kv_lora_rank
        self.qk_nope_head_dim, self.qk_rope_head_dim = qk_nope_head_dim, qk_rope_head_dim
        self.qk_head_dim = qk_nope_head_dim + qk_rope_head_dim
        self.v_head_dim = v_head_dim
        if _is_factory(attn_impl):
            assert self.qk_head_dim == v_head_dim, "SLA2 attention needs qk_head_dim == v_head_dim"
            attn_impl = attn_impl(self.qk_head_dim)
        self.attn_impl = attn_impl
        mk = partial(scaled_variance_linear, bias=False, init_constant=weight_init_constant)
        self.q_a_proj = mk(hidden_size, q_lora_rank)
        self.q_b_proj = mk(q_lora_rank, num_heads * self.qk_head_dim)
        self.kv_a_proj = mk(hidden_size, kv_lora_rank + qk_rope_head_dim)
        self.kv_b_proj = mk(kv_lora_rank, num_heads * (qk_nope_head_dim + v_head_dim))
        self.out_proj = mk(num_heads * v_head_dim, hidden_size)
        self.use_output_gate = use_output_gate
        if use_output_gate:
            self.g_proj = mk(hidden_size, num_heads * v_head_dim)
        self.q_a_layernorm = RMSNorm(q_lora_rank, eps=norm_eps)
        self.kv_a_layernorm = RMSNorm(kv_lora_rank, eps=norm_eps)
        self.q_norm = RMSNorm(qk_nope_head_dim, eps=norm_eps)
        self.k_norm = RMSNorm(qk_nope_head_dim, eps=norm_eps)

    def forward(self, x, rope_cos: Tensor, rope_sin: Tensor):
        plain = not isinstance(x, Dual)
        x = D.lift(x)
        b, l, _ = x.p.shape
        H, dq, dc = self.num_heads, self.q_lora_rank, self.kv_lora_rank
        dn, dr, dv = self.qk_nope_head_dim, self.qk_rope_head_dim, self.v_head_dim

        # one GEMM for every projection that reads x: [q_a | kv_a | g_proj]
        ws = [self.q_a_proj.weight, self.kv_a_proj.weight]
        if self.use_output_gate:
            ws.append(self.g_proj.weight)
        a = D.linear(x, torch.cat(ws, dim=0))
        q_lat = self.q_a_layernorm(a.map(lambda z: z[..., :dq]))
        kv_lat = self.kv_a_layernorm(a.map(lambda z: z[..., dq:dq + dc]))
        k_rope = a.map(lambda z: z[..., dq + dc:dq + dc + dr].unsqueeze(2))   # (b,l,1,dr)

        q = D.linear(q_lat, self.q_b_proj.weight).map(lambda z: z.reshape(b, l, H, dn + dr))
        kv = D.linear(kv_lat, self.kv_b_proj.weight).map(lambda z: z.reshape(b, l, H, dn + dv))

        q_nope = self.q_norm(q.map(lambda z: z[..., :dn]))
        k_nope = self.k_norm(kv.map(lambda z: z[..., :dn]))
        v = kv.map(lambda z: z[..., dn:])
        q_rope = D.rope(q.map(lambda z: z[..., dn:]), rope_cos, rope_sin)
        k_rope = D.rope(k_rope, rope_cos, rope_sin).map(lambda z: z.expand(b, l, H, dr))
        qf = D.cat([q_nope, q_rope], dim=-1)
        kf = D.cat([k_nope, k_rope], dim=-1)

        o = self.attn_impl(qf, kf, v).map(lambda z: z.reshape(b, l, H * dv))
        if self.use_output_gate:
            g = a.map(lambda z: z[..., dq + dc + dr:])
            o = D.sigmoid_gate(o, g)
        out = D.linear(o, self.out_proj.weight)
        return out.p if plain else out


class TransformerBlock(nn.Module):
    def __init__(self, hidden_size, num_heads, q_lora_rank, kv_lora_rank,
                 qk_nope_head_dim, qk_rope_head_dim, v_head_dim, mlp_ratio=8 / 3,
                 weight_init_constant=1.0, norm_eps=1e-6, attn_impl=sdpa_math_attention,
                 use_attn_res=False, situ_beta=4.0, situ_linear_beta=25.0,
                 mla_use_output_gate=True):
        super().__init__()
        self.norm1 = RMSNorm(hidden_size, eps=norm_eps)
        self.attn = MLAAttention(hidden_size, num_heads, q_lora_rank, kv_lora_rank,
                                 qk_nope_head_dim, qk_rope_head_dim, v_head_dim,
                                 weight_init_constant, norm_eps, attn_impl,
                                 mla_use_output_gate)
        self.norm2 = RMSNorm(hidden_size, eps=norm_eps)
        self.mlp = SwiGLUMlp(hidden_size, int(hidden_size * mlp_ratio),
                             weight_init_constant, situ_beta, situ_linear_beta)
        self.attn_scale = nn.Parameter(torch.zeros(hidden_size))
        self.mlp_scale = nn.Parameter(torch.zeros(hidden_size))
        if use_attn_res:
            self.attn_res_norm = RMSNorm(hidden_size, eps=norm_eps)
            self.mlp_res_norm = RMSNorm(hidden_size, eps=norm_eps)
            mk = partial(scaled_variance_linear, bias=False,
                         init_constant=weight_init_constant)
            self.attn_res_proj = mk(hidden_size, 1)
            self.mlp_res_proj = mk(hidden_size, 1)

    # ---- fused CUDA path (one autograd node per block, ops/block.py) ----
    def fused_geom(self):
        g = getattr(self, "_geom", None)
        if g is None:
            from ..ops.block import BlockGeom

            f = self.mlp.w1.out_features
            g = self._geom = BlockGeom(self.attn, self.norm1.weight.shape[0], f + (-f) % 8)
        return g

    def fused_ok(self, x: Tensor, compute_dtype) -> bool:
        if not (x.is_cuda and compute_dtype == torch.bfloat16 and x.dtype == torch.float32):
            return False
        from ..ops import cuda as cu

        if not (cu.available() and cu.has("block")):
            return False
        core = getattr(self.attn.attn_impl, "fused_core", None)
        if core is None and self.attn.attn_impl is not flash_jvp_attention:
            return False
        from ..ops.block import supported

        return supported(self.fused_geom())

    def fused_params(self, use_res: bool):
        """(w1, w2, gains..., bf16 weights) for ops.block.run_block.

        The bf16 weight copies (casts / concatenations of the fp32 parameters) are cached
        until a parameter's version counter moves, for gradient-free passes and also for
        passes under autograd whose weight gradients go straight into the parameters'
        gradient buffers (``GradSinks.direct``): those return no gradient for the
        matrices, so the copies need no autograd history and one set serves every pass
        of a step.  ``sinks.mats_cached`` tells the backward that this happened."""
        a, mlp = self.attn, self.mlp
        ws = [a.q_a_proj.weight, a.kv_a_proj.weight] + ([a.g_proj.weight] if a.use_output_gate else [])
        srcs = ws + [a.q_b_proj.weight, a.kv_b_proj.weight, a.out_proj.weight, mlp.w1.weight,
                     mlp.w3.weight, mlp.w2.weight]
        key = tuple(w._version for w in srcs)
        cache = getattr(self, "_wcache", None)
        grad_on = torch.is_grad_enabled()
        sinks = self.fused_sinks() if grad_on else None
        cacheable = not grad_on or sinks.direct()
        if sinks is not None:
            sinks.mats_cached = cacheable

        def build():
            bf = torch.bfloat16
            f = mlp.w1.out_features
            pad = (-f) % 8
            w1_, w3_, w2_ = mlp.w1.weight, mlp.w3.weight, mlp.w2.weight
            if pad:
                z = w1_.new_zeros(pad, w1_.shape[1])
                w13 = torch.cat([w1_, z, w3_, z], dim=0)
                w2_ = torch.nn.functional.pad(w2_, (0, pad))
            else:
                w13 = torch.cat([w1_, w3_], dim=0)
            return (torch.cat(ws, dim=0).to(bf), a.q_b_proj.weight.to(bf),
                    a.kv_b_proj.weight.to(bf), a.out_proj.weight.to(bf), w13.to(bf),
                    w2_.to(bf).contiguous())

        if not cacheable:
            mats = build()                      # autograd carries the weight gradients back
        elif cache is not None and cache[0] == key:
            mats = cache[1]
        else:
            with torch.no_grad():
                mats = build()
            self._wcache = (key, mats)
        if use_res:
            rs = (self.attn_res_norm.weight, self.attn_res_proj.weight,
                  self.mlp_res_norm.weight, self.mlp_res_proj.weight)
            rkey = tuple(w._version for w in rs)
            rc = getattr(self, "_rcache", None)
            if not grad_on and rc is not None and rc[0] == rkey:
                w1, w2 = rc[1]
            else:
                w1 = rs[0] * rs[1].reshape(-1)
                w2 = rs[2] * rs[3].reshape(-1)
                if not grad_on:
                    self._rcache = (rkey, (w1, w2))
        else:
            w1 = w2 = None
        return (w1, w2, self.norm1.weight, self.norm2.weight, a.q_a_layernorm.weight,
                a.kv_a_layernorm.weight, a.q_norm.weight, a.k_norm.weight, self.attn_scale,
                self.mlp_scale) + mats

    def fused_sinks(self):
        """Which parameter each row band of the six fused bf16 matrices comes from (same
        order as ``fused_params`` concatenates them), for direct weight-gradient writes."""
        sk = getattr(self, "_sinks", None)
        if sk is None:
            from ..ops.block import GradSinks

            a, mlp = self.attn, self.mlp
            ws = [a.q_a_proj.weight, a.kv_a_proj.weight] + \
                ([a.g_proj.weight] if a.use_output_gate else [])
            wa, r = [], 0
            for w in ws:
                wa.append((w, r, w.shape[0], w.shape[1]))
                r += w.shape[0]
            one = lambda w: [(w, 0, w.shape[0], w.shape[1])]
            f = mlp.w1.out_features
            fp = f + (-f) % 8
            sk = self._sinks = GradSinks({
                "W_a": wa, "W_qb": one(a.q_b_proj.weight), "W_kvb": one(a.kv_b_proj.weight),
                "W_out": one(a.out_proj.weight),
                "W13": [(mlp.w1.weight, 0, f, mlp.w1.weight.shape[1]),
                        (mlp.w3.weight, fp, f, mlp.w3.weight.shape[1])],
                "W2": [(mlp.w2.weight, 0, mlp.w2.weight.shape[0], f)]},
                small={"g_n1": self.norm1.weight, "g_n2": self.norm2.weight,
                       "g_qa": a.q_a_layernorm.weight, "g_kva": a.kv_a_layernorm.weight,
                       "g_qn": a.q_norm.weight, "g_kn": a.k_norm.weight,
                       "a_scale": self.attn_scale, "m_scale": self.mlp_scale})
        return sk

    def fused_forward(self, prefix: Dual, snaps, fresh: bool, use_res: bool, rope_cos, rope_sin,
                      eps: float) -> Dual:
        from ..ops.block import DENSE_CORE, run_block

        core = getattr(self.attn.attn_impl, "fused_core", None) or DENSE_CORE
        act = self.mlp.act
        has_t = prefix.t is not None
        p, t = run_block(self.fused_geom(), core, fresh, use_res, eps, act.beta, act.linear_beta,
                         rope_cos, rope_sin, prefix.p, prefix.t, [s.p for s in snaps],
                         [s.t for s in snaps] if has_t else [None] * len(snaps),
                         self.fused_params(use_res),
                         self.fused_sinks() if torch.is_grad_enabled() else None)
        return Dual(p, t)

    def forward(self, x, rope_cos, rope_sin, compute_dtype=None):
        """Plain pre-norm block (no attention residual)."""
        plain = not isinstance(x, Dual)
        x = D.lift(x)
        if self.fused_ok(x.p, compute_dtype):
            out = self.fused_forward(x, [], False, False, rope_cos, rope_sin, self.norm1.eps)
            return out.p if plain else out
        a = self.attn(self.norm1(x, compute_dtype), rope_cos, rope_sin)
        x = D.scale_add(x, a, self.attn_scale)
        m = self.mlp(self.norm2(x, compute_dtype))
        x = D.scale_add(x, m, self.mlp_scale)
        return x.p if plain else x


class FinalLayer(nn.Module):
    def __init__(self, hidden_size, patch_size, out_channels, norm_eps=1e-6):
        super().__init__()
        pt, ph, pw = patch_size
        self.norm = RMSNorm(hidden_size, eps=norm_eps)
        self.linear = nn.Linear(hidden_size, pt * ph * pw * out_channels, bias=True)
        with torch.no_grad():
            self.linear.weight.zero_()
            self.linear.bias.zero_()

    def forward(self, x, compute_dtype=None):
        plain = not isinstance(x, Dual)
        y = D.linear(self.norm(D.lift(x), compute_dtype), self.linear.weight, self.linear.bias)
        return y.p if plain else y


# ------------------------------------------------------------------ rope ---
def precompute_axial_rope_3d(head_dim: int, grid_size, num_prefix_tokens: int,
                             axis_dims=None, theta: float = 10000.0):
    """cos/sin tables (prefix + T*Gh*Gw, head_dim/2): the rotary band is split
    over (t, h, w) as about (1/4, 3/8, 3/8), each an even number of channels;
    prefix tokens get angle 0 (reference ``models/imf_dit_video.py:557-602``)."""
    if axis_dims is None:
        dt = 2 * ((head_dim // 4) // 2)
        dh = 2 * (((head_dim - dt) // 2) // 2)
        axis_dims = (dt, dh, head_dim - dt - dh)
    assert sum(axis_dims) == head_dim and all(a % 2 == 0 for a in axis_dims)
    gt, gh, gw = grid_size
    pos = torch.meshgrid(torch.arange(gt, dtype=torch.float32),
                         torch.arange(gh, dtype=torch.float32),
                         torch.arange(gw, dtype=torch.float32), indexing="ij")
    cols = []
    for p, ad in zip(pos, axis_dims):
        inv = 1.0 / (theta ** (torch.arange(0, ad, 2, dtype=torch.float32) / ad))
        cols.append(p.reshape(-1, 1) * inv[None, :])
    ang = torch.cat(cols, dim=-1)
    ang = torch.cat([torch.zeros(num_prefix_tokens, head_dim // 2), ang], dim=0)
    return torch.cos(ang), torch.sin(ang)


# ------------------------------------------------- dual checkpointing -----
class _CheckpointDual(torch.autograd.Function):
    """Activation checkpoint for a dual-number segment.

    Forward runs ``fn`` on (primal, tangent) inputs without a graph and keeps
    only the primal inputs.  Backward re-runs ``fn`` PRIMAL-ONLY (tangents
    are never differentiated, so the expensive tangent half is not
    recomputed) and backpropagates through that; parameter gradients
    accumulate directly into ``.grad``.  Counterpart of the reference's
    per-block functional checkpoint (``models/imf_dit_video.py:909-972``)."""

    @staticmethod
    def forward(ctx, fn, n_primal, *tensors):
        ctx.fn = fn
        prim = tensors[:n_primal]
        tang = tensors[n_primal:]
        ctx.save_for_backward(*prim)
        with torch.no_grad():
            out = fn([Dual(p.detach(), None if t is None else t)
                      for p, t in zip(prim, tang)])
        ctx.has_t = out.t is not None
        if out.t is not None:
            ctx.mark_non_differentiable(out.t)
            return out.p, out.t
        return out.p, out.p.new_empty(0)

    @staticmethod
    def backward(ctx, gp, _gt):
        prim = [p.detach().requires_grad_(p.requires_grad or True) for p in ctx.saved_tensors]
        with torch.enable_grad():
            out = ctx.fn([Dual(p, None) for p in prim])
        torch.autograd.backward(out.p, gp)
        return (None, None) + tuple(p.grad for p in prim) + (None,) * len(prim)


def checkpoint_dual(fn: Callable[[List[Dual]], Dual], inputs: Sequence[Dual]) -> Dual:
    prim = [x.p for x in inputs]
    tang = [x.t for x in inputs]
    p, t = _CheckpointDual.apply(fn, len(prim), *prim, *tang)
    return Dual(p, t if t.numel() or p.numel() == 0 else None)


# ----------------------------------------------------------------- model ---
class IMFDiTVideo(nn.Module):
    """improved-MeanFlow video DiT: shared trunk (depth - aux) + u branch (aux)
    + v branch (aux; absent in eval_mode)."""

    def __init__(self, input_size=16, num_frames=3, patch_size=(1, 2, 2), in_channels=16,
                 hidden_size=768, depth=12, num_heads=12, mlp_ratio=8 / 3, num_classes=1000,
                 aux_head_depth=8, q_lora_rank=0, kv_lora_rank=0, qk_nope_head_dim=0,
                 qk_rope_head_dim=0, v_head_dim=0, num_class_tokens=8, num_time_tokens=4,
                 num_cfg_tokens=4, num_interval_tokens=2, freq_embedding_size=256,
                 token_init_constant=1.0, embedding_init_constant=1.0,
                 weight_init_constant=0.32, rmsnorm_eps=1e-6, rope_theta=10000.0,
                 attn_impl=sdpa_math_attention, eval_mode=False, attn_res_block_size=0,
                 situ_beta=4.0, situ_linear_beta=25.0, mla_use_output_gate=True,
                 grad_checkpoint=False, compute_dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.head_dim = hidden_size // num_heads
        self.attn_res_block_size = attn_res_block_size
        self.grad_checkpoint = grad_checkpoint
        self.compute_dtype = compute_dtype
        self.rmsnorm_eps = rmsnorm_eps
        hd = self.head_dim
        # MLA geometry defaults (reference ``models/imf_dit_video.py:661-676``)
        self.v_head_dim = v_head_dim or hd
        self.qk_rope_head_dim = qk_rope_head_dim or max(2, hd // 4)
        self.qk_nope_head_dim = qk_nope_head_dim or hd - self.qk_rope_head_dim
        self.qk_head_dim = self.qk_nope_head_dim + self.qk_rope_head_dim
        self.q_lora_rank = q_lora_rank or max(hd, hidden_size // 2)
        self.kv_lora_rank = kv_lora_rank or max(hd, hidden_size // 4)
        assert self.qk_rope_head_dim % 2 == 0 and self.qk_nope_head_dim % 2 == 0

        self.patch_size = tuple(patch_size)
        self.in_channels = self.out_channels = in_channels
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.eval_mode = eval_mode
        pt, ph, pw = self.patch_size
        in_h, in_w = (input_size, input_size) if isinstance(input_size, int) else input_size
        self.grid_size = (num_frames // pt, in_h // ph, in_w // pw)
        num_patches = self.grid_size[0] * self.grid_size[1] * self.grid_size[2]

        self.x_embedder = VideoPatchEmbedder(in_channels, hidden_size, self.patch_size, True)
        te = dict(hidden_size=hidden_size, frequency_embedding_size=freq_embedding_size,
                  init_constant=embedding_init_constant)
        self.h_embedder = TimestepEmbedder(**te)
        self.omega_embedder = TimestepEmbedder(**te)
        self.cfg_t_start_embedder = TimestepEmbedder(**te)
        self.cfg_t_end_embedder = TimestepEmbedder(**te)
        self.y_embedder = LabelEmbedder(num_classes, hidden_size, embedding_init_constant)

        std = token_init_constant / math.sqrt(hidden_size)
        self.time_tokens = nn.Parameter(torch.randn(num_time_tokens, hidden_size) * std)
        self.class_tokens = nn.Parameter(torch.randn(num_class_tokens, hidden_size) * std)
        self.omega_tokens = nn.Parameter(torch.randn(num_cfg_tokens, hidden_size) * std)
        self.t_min_tokens = nn.Parameter(torch.randn(num_interval_tokens, hidden_size) * std)
        self.t_max_tokens = nn.Parameter(torch.randn(num_interval_tokens, hidden_size) * std)
        self.prefix_tokens = (num_class_tokens + num_cfg_tokens
                              + 2 * num_interval_tokens + num_time_tokens)
        self.seq_len = self.prefix_tokens + num_patches

        cos, sin = precompute_axial_rope_3d(self.qk_rope_head_dim, self.grid_size,
                                            self.prefix_tokens, theta=rope_theta)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

        # module-factory attention (SLA2 family): bind sequence length and head
        # count; cube attention keeps the whole forward in 3-D-tile token order
        self.tile_major = False
        if isinstance(attn_impl, partial) and isinstance(attn_impl.func, type):
            attn_impl = partial(attn_impl, seq_len=self.seq_len, num_heads=num_heads)
            if getattr(attn_impl.func, "TILE_MAJOR", False):
                from .sla2 import tile_permutation

                tile = attn_impl.keywords.get("tile", (4, 4, 4))
                perm, inv, _ = tile_permutation(self.grid_size, tile, self.prefix_tokens)
                self.register_buffer("tm_perm", perm, persistent=False)
                self.register_buffer("tm_inv", inv, persistent=False)
                self.tile_major = True
                attn_impl = partial(attn_impl, pre_permuted=True)
                self.rope_cos = self.rope_cos[perm]
                self.rope_sin = self.rope_sin[perm]

        kw = dict(hidden_size=hidden_size, num_heads=num_heads, q_lora_rank=self.q_lora_rank,
                  kv_lora_rank=self.kv_lora_rank, qk_nope_head_dim=self.qk_nope_head_dim,
                  qk_rope_head_dim=self.qk_rope_head_dim, v_head_dim=self.v_head_dim,
                  mlp_ratio=mlp_ratio, weight_init_constant=weight_init_constant,
                  norm_eps=rmsnorm_eps, attn_impl=attn_impl,
                  use_attn_res=attn_res_block_size > 0, situ_beta=situ_beta,
                  situ_linear_beta=situ_linear_beta, mla_use_output_gate=mla_use_output_gate)
        shared_depth = depth - aux_head_depth
        self.shared_blocks = nn.ModuleList(TransformerBlock(**kw) for _ in range(shared_depth))
        self.u_heads = nn.ModuleList(TransformerBlock(**kw) for _ in range(aux_head_depth))
        self.v_heads = nn.ModuleList(
            TransformerBlock(**kw) for _ in range(0 if eval_mode else aux_head_depth))
        self.u_final_layer = FinalLayer(hidden_size, self.patch_size, in_channels, rmsnorm_eps)
        self.v_final_layer = FinalLayer(hidden_size, self.patch_size, in_channels, rmsnorm_eps)
        if attn_res_block_size > 0:
            mk = partial(scaled_variance_linear, bias=False,
                         init_constant=weight_init_constant)
            self.u_out_res_norm = RMSNorm(hidden_size, eps=rmsnorm_eps)
            self.v_out_res_norm = RMSNorm(hidden_size, eps=rmsnorm_eps)
            self.u_out_res_proj = mk(hidden_size, 1)
            self.v_out_res_proj = mk(hidden_size, 1)

    # ------------------------------------------------------------ pieces ---
    def _use_ckpt(self) -> bool:
        return (self.grad_checkpoint and torch.is_grad_enabled()
                and not torch._C._are_functorch_transforms_active())

    def unpatchify(self, x: Tensor) -> Tensor:
        """(B, N, pt*ph*pw*C) bf16 / fp32 -> (B, C, T, H, W) fp32 (one scatter kernel on CUDA)."""
        from ..ops.patch import unpatch_rows

        pt, ph, pw = self.patch_size
        gt, gh, gw = self.grid_size
        assert gt * gh * gw == x.shape[1]
        shape = (x.shape[0], self.out_channels, gt * pt, gh * ph, gw * pw)
        return unpatch_rows(x, shape, self.patch_size, c_last=True)

    def _build_sequence(self, x, h, w, t_min, t_max, y) -> Dual:
        """[class | omega | t_min | t_max | time | patches]; omega enters as
        1 - 1/omega; t itself is not an input, only h = t - r."""
        x, h = D.lift(x), D.lift(h)
        xe = self.x_embedder(x)
        he = self.h_embedder(h)
        oe = self.omega_embedder(1 - 1 / w).p
        lo = self.cfg_t_start_embedder(t_min).p
        hi = self.cfg_t_end_embedder(t_max).p
        ye = self.y_embedder(y)
        bank = lambda tok, e: tok + e.unsqueeze(1)
        time_p = bank(self.time_tokens, he.p)
        parts = [bank(self.class_tokens, ye), bank(self.omega_tokens, oe),
                 bank(self.t_min_tokens, lo), bank(self.t_max_tokens, hi), time_p]
        dt = torch.float32 if self.compute_dtype is not None else xe.p.dtype
        p = torch.cat([z.to(dt) for z in parts] + [xe.p.to(dt)], dim=1)
        t = None
        if xe.t is not None or he.t is not None:
            with torch.no_grad():
                nt = self.time_tokens.shape[0]
                n0 = self.prefix_tokens - nt
                b = p.shape[0]
                z0 = p.new_zeros(b, n0, p.shape[-1])
                tt = (he.t.unsqueeze(1).expand(b, nt, -1).to(dt) if he.t is not None
                      else p.new_zeros(b, nt, p.shape[-1]))
                xt = xe.t.to(dt) if xe.t is not None else torch.zeros_like(xe.p, dtype=dt)
                t = torch.cat([z0, tt, xt], dim=1)
        return Dual(p, t)

    def _res_block(self, blk: TransformerBlock, fresh: bool, prefix: Dual,
                   snaps: List[Dual]) -> Dual:
        eps, cd = self.rmsnorm_eps, self.compute_dtype
        if blk.fused_ok(prefix.p, cd):
            return blk.fused_forward(prefix, snaps, fresh, True, self.rope_cos, self.rope_sin, eps)
        h1 = (D.attn_res(prefix, snaps, blk.attn_res_norm.weight, blk.attn_res_proj.weight, eps)
              if snaps else prefix)
        a = blk.attn(blk.norm1(h1, cd), self.rope_cos, self.rope_sin)
        if fresh:
            snaps2, p2 = snaps + [prefix], D.scale_add(None, a, blk.attn_scale)
            p2 = Dual(p2.p.to(prefix.p.dtype), None if p2.t is None else p2.t.to(prefix.p.dtype))
        else:
            snaps2, p2 = snaps, D.scale_add(prefix, a, blk.attn_scale)
        h2 = D.attn_res(p2, snaps2, blk.mlp_res_norm.weight, blk.mlp_res_proj.weight, eps)
        m = blk.mlp(blk.norm2(h2, cd))
        return D.scale_add(p2, m, blk.mlp_scale)

    def _run_attn_res_blocks(self, prefix: Dual, snaps: List[Dual], blocks, start_idx: int):
        """Attention-residual schedule with a global block index: every
        ``attn_res_block_size`` blocks the running prefix sum is snapshotted
        and restarted from that block's gated attention output."""
        bs = self.attn_res_block_size
        snaps = list(snaps)
        for j, blk in enumerate(blocks):
            fresh = (start_idx + j) % bs == 0
            if self._use_ckpt():
                fn = lambda xs, blk=blk, fresh=fresh: self._res_block(blk, fresh, xs[0], xs[1:])
                new_prefix = checkpoint_dual(fn, [prefix] + snaps)
            else:
                new_prefix = self._res_block(blk, fresh, prefix, snaps)
            if fresh:
                snaps = snaps + [prefix]
            prefix = new_prefix
        return prefix, snaps

    def _run_plain_blocks(self, seq: Dual, blocks) -> Dual:
        for blk in blocks:
            if self._use_ckpt():
                fn = lambda xs, blk=blk: blk(xs[0], self.rope_cos, self.rope_sin,
                                             self.compute_dtype)
                seq = checkpoint_dual(fn, [seq])
            else:
                seq = blk(seq, self.rope_cos, self.rope_sin, self.compute_dtype)
        return seq

    def _fused_out_head_ok(self, pf: Dual, sn) -> bool:
        """Output re-mix + final RMSNorm in one kernel: bf16 compute on the kernel library,
        fp32 (B, L, d) streams, d a multiple of 128."""
        if self.compute_dtype != torch.bfloat16 or not pf.p.is_cuda or pf.p.dtype != torch.float32:
            return False
        if pf.p.shape[-1] % 128 or len(sn) + 1 > 8:
            return False
        try:
            from ..ops import cuda as cu
            return cu.available() and cu.has("block")
        except Exception:
            return False

    def _fused_head(self, pf: Dual, sn, gain, pw, final: FinalLayer, keep_tangent: bool):
        from ..ops.block import out_head

        w = gain.float() * pw.reshape(-1).float()
        if not keep_tangent:
            pf, sn = Dual(pf.p, None), [Dual(s.p, None) for s in sn]
        n, dn = out_head(pf, sn, w, final.norm.weight, final.norm.eps)
        seq = Dual(n, dn)
        if self.tile_major:
            seq = seq.map(lambda z: permute_rows(z, self.tm_inv, self.tm_perm))
        tok = seq.map(lambda z: z[:, self.prefix_tokens:])
        y = D.linear(tok, final.linear.weight, final.linear.bias)
        return y.map(self.unpatchify)

    def _head(self, seq: Dual, final: FinalLayer, keep_tangent: bool):
        if self.tile_major:
            seq = seq.map(lambda z: permute_rows(z, self.tm_inv, self.tm_perm))
        tok = seq.map(lambda z: z[:, self.prefix_tokens:])
        if not keep_tangent:
            tok = Dual(tok.p, None)
        out = final(tok, self.compute_dtype).map(self.unpatchify)
        return out

    # ----------------------------------------------------------- forward ---
    def forward_dual(self, x, h, w, t_min, t_max, y, branches: Sequence[str] = ("u", "v"),
                     tangent_branches: Sequence[str] = ("u",)):
        """Evaluate on dual numbers.

        Args:
            x: Dual (B, C, T, H, W) latents (+ tangent);  h: Dual (B,) = t - r.
            w, t_min, t_max: (B,) guidance scale / interval;  y: (B,) labels.
            branches: which output branches to run ("u", "v").
            tangent_branches: branches whose tangent is propagated past the
                shared trunk (iMF needs du/dt only; the v branch stays primal).

        Returns: dict branch -> Dual (B, C, T, H, W), fp32.
        """
        x, h = D.lift(x), D.lift(h)
        if len(self.v_heads) == 0:
            branches = [b for b in branches if b == "u"] or ["u"]
        seq = self._build_sequence(x, h, w, t_min, t_max, y)
        if self.tile_major:
            seq = seq.map(lambda z: permute_rows(z, self.tm_perm, self.tm_inv))
        need_t = seq.t is not None and any(b in tangent_branches for b in branches)
        if not need_t:
            seq = Dual(seq.p, None)
        out = {}
        if self.attn_res_block_size > 0:
            sd = len(self.shared_blocks)
            prefix, snaps = self._run_attn_res_blocks(seq, [], self.shared_blocks, 0)
            for name, heads, norm, proj, final in (
                    ("u", self.u_heads, "u_out_res_norm", "u_out_res_proj", self.u_final_layer),
                    ("v", self.v_heads, "v_out_res_norm", "v_out_res_proj", self.v_final_layer)):
                if name not in branches:
                    continue
                kt = need_t and name in tangent_branches
                pf, sn = (prefix, snaps) if kt else (
                    Dual(prefix.p, None), [Dual(s.p, None) for s in snaps])
                pf, sn = self._run_attn_res_blocks(pf, sn, heads, sd)
                gain, pw = getattr(self, norm).weight, getattr(self, proj).weight
                if self._use_ckpt():
                    fn = lambda xs, gain=gain, pw=pw: D.attn_res(xs[0], xs[1:], gain, pw,
                                                                 self.rmsnorm_eps)
                    s = checkpoint_dual(fn, [pf] + sn)
                else:
                    if self._fused_out_head_ok(pf, sn):
                        out[name] = self._fused_head(pf, sn, gain, pw, final, kt)
                        continue
                    s = D.attn_res(pf, sn, gain, pw, self.rmsnorm_eps)
                out[name] = self._head(s, final, kt)
        else:
            seq = self._run_plain_blocks(seq, self.shared_blocks)
            for name, heads, final in (("u", self.u_heads, self.u_final_layer),
                                       ("v", self.v_heads, self.v_final_layer)):
                if name not in branches:
                    continue
                kt = need_t and name in tangent_branches
                s = self._run_plain_blocks(seq if kt else Dual(seq.p, None), heads)
                out[name] = self._head(s, final, kt)
        return out

    def forward(self, x, t, h, w, t_min, t_max, y):
        """Reference-compatible entry: returns (u, v), each (B, C, T, H, W)."""
        out = self.forward_dual(Dual(x), Dual(h), w, t_min, t_max, y)
        u = out["u"].p
        v = out["v"].p if "v" in out else u
        return u, v


def imf_dit_video_S(num_classes, **kw):
    return IMFDiTVideo(hidden_size=384, depth=8, num_heads=6, aux_head_depth=4,
                       num_classes=num_classes, **kw)


def imf_dit_video_B(num_classes, **kw):
    return IMFDiTVideo(hidden_size=768, depth=12, num_heads=12, aux_head_depth=8,
                       num_classes=num_classes, **kw)
