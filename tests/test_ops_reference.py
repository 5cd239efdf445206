"""CPU: every hand-written tangent formula against torch.func.jvp of the
primal formula (the oracle the CUDA kernels are later compared with)."""
import math

import pytest
import torch

from imfvideo_b200.ops import reference as ref


def _jvp(fn, xs, ts):
    return torch.func.jvp(fn, tuple(xs), tuple(ts))


@pytest.mark.parametrize("shape", [(3, 5, 64), (2, 7, 48)])
def test_rmsnorm_jvp(shape):
    torch.manual_seed(0)
    x, dx = torch.randn(shape, dtype=torch.float64), torch.randn(shape, dtype=torch.float64)
    w = torch.rand(shape[-1], dtype=torch.float64) + 0.5
    y0, dy0 = _jvp(lambda a: ref.rmsnorm(a, w, 1e-5), [x], [dx])
    y, dy = ref.rmsnorm_jvp(x.float(), dx.float(), w.float(), 1e-5)
    assert torch.allclose(y.double(), y0, atol=1e-5)
    assert torch.allclose(dy.double(), dy0, atol=1e-5)


@pytest.mark.parametrize("lb", [None, 25.0, 2.0])
def test_situ_jvp(lb):
    torch.manual_seed(1)
    g, u, dg, du = (torch.randn(4, 9, 33) * 3 for _ in range(4))
    y0, dy0 = _jvp(lambda a, b: ref.situ_mul(a, b, 4.0, lb), [g, u], [dg, du])
    y, dy = ref.situ_mul_jvp(g, u, dg, du, 4.0, lb)
    assert torch.allclose(y, y0, atol=1e-5) and torch.allclose(dy, dy0, atol=2e-5)


@pytest.mark.parametrize("J", [1, 2, 6])
def test_attn_res_jvp(J):
    torch.manual_seed(2)
    cands = [torch.randn(2, 11, 32) for _ in range(J)]
    dc = [torch.randn(2, 11, 32) for _ in range(J)]
    w = torch.randn(32)
    f = lambda *cs: ref.attn_res(list(cs), w, 1e-6)
    y0, dy0 = _jvp(f, cands, dc)
    y, dy = ref.attn_res_jvp(cands, dc, w, 1e-6)
    assert torch.allclose(y, y0, atol=1e-5) and torch.allclose(dy, dy0, atol=1e-5)


@pytest.mark.parametrize("L,dk,dv", [(37, 16, 16), (64, 24, 8)])
def test_attention_jvp(L, dk, dv):
    torch.manual_seed(3)
    q, k, dq, dk_ = (torch.randn(2, L, 3, dk) for _ in range(4))
    v, dv_ = torch.randn(2, L, 3, dv), torch.randn(2, L, 3, dv)
    o0, do0 = _jvp(ref.attention, [q, k, v], [dq, dk_, dv_])
    o, do = ref.attention_jvp(q, k, v, dq, dk_, dv_, chunk=16)
    assert torch.allclose(o, o0, atol=1e-5) and torch.allclose(do, do0, atol=1e-5)
    sd = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
    assert torch.allclose(o, sd, atol=1e-5)
    lse = ref.attention_lse(q, k)
    assert lse.shape == (2, 3, L) and torch.isfinite(lse).all()


def test_rope_linear_and_norm_preserving():
    torch.manual_seed(4)
    x = torch.randn(2, 10, 3, 16)
    ang = torch.rand(10, 8) * 6
    y = ref.rope(x, torch.cos(ang), torch.sin(ang))
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    y2 = ref.rope(2 * x, torch.cos(ang), torch.sin(ang))
    assert torch.allclose(y2, 2 * y, atol=1e-5)


def test_newton_schulz_reference_orthogonalises():
    torch.manual_seed(5)
    G = torch.randn(48, 96)
    X = ref.newton_schulz(G, (3.4445, -4.7750, 2.0315), steps=5)
    s = torch.linalg.svdvals(X)
    assert s.min() > 0.5 and s.max() < 1.3
