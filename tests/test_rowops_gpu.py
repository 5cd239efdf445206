"""GPU: fused per-token kernels (forward, tangent, backward) against the
plain-PyTorch fp32 formulas and autograd."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16, F32 = torch.bfloat16, torch.float32


@pytest.fixture(scope="module")
def R():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from imfvideo_b200.ops import cuda as cu

    assert cu.available()
    from imfvideo_b200.ops import rowops

    return rowops


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _rn(*shape, dt=F32, s=1.0):
    return (torch.randn(*shape, device="cuda") * s).to(dt)


def _resnorm_ref(res, y, gate, snaps, w, gain, eps):
    from imfvideo_b200.ops import reference as ref

    pfx = (res if res is not None else 0) + (y.float() * gate if y is not None else 0)
    h = ref.attn_res(list(snaps) + [pfx], w, eps) if w is not None else pfx
    return pfx, ref.rmsnorm(h, gain, eps)


@pytest.mark.parametrize("D,ns,with_y,with_res,with_w", [
    (256, 0, False, True, False), (256, 2, True, True, True), (256, 4, True, False, True),
    (1024, 1, True, True, True), (128, 0, True, True, True)])
def test_resnorm_forward_tangent_backward(R, D, ns, with_y, with_res, with_w):
    torch.manual_seed(D + ns)
    rows, eps = 203, 1e-5
    res, dres = (_rn(rows, D), _rn(rows, D)) if with_res else (None, None)
    y, dy = (_rn(rows, D, dt=BF16), _rn(rows, D, dt=BF16)) if with_y else (None, None)
    gate = _rn(D) if with_y else None
    snaps, dsn = [_rn(rows, D) for _ in range(ns)], [_rn(rows, D) for _ in range(ns)]
    w = _rn(D, s=0.2) if with_w else None
    gain = torch.rand(D, device="cuda") + 0.5
    n, dn = torch.empty(rows, D, dtype=BF16, device="cuda"), torch.empty(rows, D, dtype=BF16, device="cuda")
    pfx = torch.empty(rows, D, device="cuda") if with_y else None
    dpfx = torch.empty(rows, D, device="cuda") if with_y else None
    R.resnorm_fwd(res, dres, y, dy, gate, snaps, dsn, w, gain, eps, n, dn, pfx, dpfx)
    # oracle: forward-mode through the formulas
    prim = [t for t in [res, y.float() if with_y else None] + snaps if t is not None]
    tang = [t for t in [dres, dy.float() if with_y else None] + dsn if t is not None]

    def f(*xs):
        xs = list(xs)
        r_ = xs.pop(0) if with_res else None
        y_ = xs.pop(0) if with_y else None
        return _resnorm_ref(r_, y_, gate, xs, w, gain, eps)
    (pfx0, n0), (dpfx0, dn0) = torch.func.jvp(f, tuple(prim), tuple(tang))
    assert _rel(n, n0) < 6e-3 and _rel(dn, dn0) < 6e-3
    if with_y:
        assert _rel(pfx, pfx0) < 1e-6 and _rel(dpfx, dpfx0) < 1e-6
    # reverse mode
    gn = _rn(rows, D, dt=BF16)
    gext = _rn(rows, D)
    leaves = [t.clone().requires_grad_(True) for t in prim]
    gate_l = gate.clone().requires_grad_(True) if with_y else None
    w_l = w.clone().requires_grad_(True) if with_w else None
    gain_l = gain.clone().requires_grad_(True)
    xs = list(leaves)
    r_ = xs.pop(0) if with_res else None
    y_ = xs.pop(0) if with_y else None
    pr, nr = _resnorm_ref(r_, y_, gate_l, xs, w_l, gain_l, eps)
    ((nr * gn.float()).sum() + (pr * gext).sum()).backward()
    g_res, g_y, g_sn, g_gain, g_w, g_gate = R.resnorm_bwd(res, y, gate, snaps, w, gain, eps, gn, gext)
    i = 0
    if with_res:
        assert _rel(g_res, leaves[i].grad) < 1e-4
        i += 1
    if with_y:
        assert _rel(g_y, leaves[i].grad) < 6e-3
        assert _rel(g_gate, gate_l.grad) < 1e-4
        i += 1
    for j in range(ns):
        assert _rel(g_sn[j], leaves[i + j].grad) < 1e-4
    assert _rel(g_gain, gain_l.grad) < 1e-4
    if with_w and (ns > 0):
        assert _rel(g_w, w_l.grad) < 1e-3


def test_rmsnorm_segments(R):
    from imfvideo_b200.ops import reference as ref

    torch.manual_seed(0)
    rows, dq, dc, na, eps = 301, 128, 64, 272, 1e-5
    a, da = _rn(rows, na, dt=BF16), _rn(rows, na, dt=BF16)
    g1, g2 = torch.rand(dq, device="cuda") + 0.5, torch.rand(dc, device="cuda") + 0.5
    o1, do1 = torch.empty(rows, dq, dtype=BF16, device="cuda"), torch.empty(rows, dq, dtype=BF16, device="cuda")
    o2, do2 = torch.empty(rows, dc, dtype=BF16, device="cuda"), torch.empty(rows, dc, dtype=BF16, device="cuda")
    R.rmsnorm_seg_fwd([(a, da, g1, o1, do1, dq, na, dq),
                       (a[:, dq:], da[:, dq:], g2, o2, do2, dc, na, dc)], rows, eps, True)
    for (x, dx, g, o, do) in ((a[:, :dq], da[:, :dq], g1, o1, do1),
                              (a[:, dq:dq + dc], da[:, dq:dq + dc], g2, o2, do2)):
        y0, dy0 = ref.rmsnorm_jvp(x.float(), dx.float(), g, eps)
        assert _rel(o, y0) < 5e-3 and _rel(do, dy0) < 5e-3
    gy1, gy2 = _rn(rows, dq, dt=BF16), _rn(rows, dc, dt=BF16)
    gx = torch.zeros(rows, na, dtype=BF16, device="cuda")
    gg1, gg2 = R.rmsnorm_seg_bwd([(a, g1, gy1, gx, dq, na, dq),
                                  (a[:, dq:], g2, gy2, gx[:, dq:], dc, na, dc)], rows, eps)
    xl = a.float().requires_grad_(True)
    g1l, g2l = g1.clone().requires_grad_(True), g2.clone().requires_grad_(True)
    (ref.rmsnorm(xl[:, :dq], g1l, eps) * gy1.float()).sum().backward()
    (ref.rmsnorm(xl[:, dq:dq + dc], g2l, eps) * gy2.float()).sum().backward()
    assert _rel(gx[:, :dq + dc], xl.grad[:, :dq + dc]) < 6e-3
    assert _rel(gg1, g1l.grad) < 1e-4 and _rel(gg2, g2l.grad) < 1e-4
    assert (gx[:, dq + dc:] == 0).all()


def _prep_ref(qb, kvb, kr, cos, sin, qg, kg, B, L, H, dn, dr, dv, eps):
    from imfvideo_b200.ops import reference as ref

    q = qb.reshape(B, L, H, dn + dr)
    kv = kvb.reshape(B, L, H, dn + dv)
    qn = ref.rmsnorm(q[..., :dn], qg, eps)
    kn = ref.rmsnorm(kv[..., :dn], kg, eps)
    qr = ref.rope(q[..., dn:], cos, sin)
    krr = ref.rope(kr.reshape(B, L, 1, dr), cos, sin).expand(B, L, H, dr)
    return torch.cat([qn, qr], -1), torch.cat([kn, krr], -1)


@pytest.mark.parametrize("H,dn,dr,dv", [(4, 48, 16, 64), (5, 48, 16, 64), (3, 96, 32, 128),
                                        (12, 64, 64, 128), (2, 44, 20, 64)])
def test_qk_prep(R, H, dn, dr, dv):
    """(4, 48, 16, 64): the model's geometry; 5 heads: a last pass with one live head of four;
    head_dim 128: two heads per warp pass; (2, 44, 20, 64): not 8-aligned, the narrow kernels."""
    torch.manual_seed(0)
    B, L, eps = 2, 77, 1e-5
    hd = dn + dr
    rows, na = B * L, 8 + dr + 16
    qb, dqb = _rn(rows, H * hd, dt=BF16), _rn(rows, H * hd, dt=BF16)
    kvb, dkvb = _rn(rows, H * (dn + dv), dt=BF16), _rn(rows, H * (dn + dv), dt=BF16)
    a, da = _rn(rows, na, dt=BF16), _rn(rows, na, dt=BF16)
    kr, dkr = a[:, 8:8 + dr], da[:, 8:8 + dr]
    ang = torch.rand(L, dr // 2, device="cuda") * 6
    cos, sin = torch.cos(ang), torch.sin(ang)
    qg, kg = torch.rand(dn, device="cuda") + 0.5, torch.rand(dn, device="cuda") + 0.5
    mk = lambda: torch.empty(B, L, H, hd, dtype=BF16, device="cuda")
    q, dq, k, dk = mk(), mk(), mk(), mk()
    R.qkprep_fwd(qb, dqb, kvb, dkvb, kr, dkr, cos, sin, qg, kg, q, dq, k, dk, rows, L, H, dn, dr,
                 dv, na, eps)
    f = lambda a_, b_, c_: _prep_ref(a_, b_, c_, cos, sin, qg, kg, B, L, H, dn, dr, dv, eps)
    (q0, k0), (dq0, dk0) = torch.func.jvp(f, (qb.float(), kvb.float(), kr.float()),
                                          (dqb.float(), dkvb.float(), dkr.float()))
    for x, x0 in ((q, q0), (dq, dq0), (k, k0), (dk, dk0)):
        assert _rel(x, x0) < 5e-3
    # backward
    gq, gk = _rn(B, L, H, hd, dt=BF16), _rn(B, L, H, hd, dt=BF16)
    g_qb = torch.empty_like(qb)
    g_kvb = torch.zeros_like(kvb)
    g_a = torch.zeros_like(a)
    ggq, ggk = R.qkprep_bwd(qb, kvb, cos, sin, qg, kg, gq, gk, g_qb, g_kvb, g_a[:, 8:], rows, L, H,
                            dn, dr, dv, na, eps)
    ql, kvl, krl = (t.float().requires_grad_(True) for t in (qb, kvb, kr))
    qgl, kgl = qg.clone().requires_grad_(True), kg.clone().requires_grad_(True)
    qq, kk = _prep_ref(ql, kvl, krl, cos, sin, qgl, kgl, B, L, H, dn, dr, dv, eps)
    ((qq * gq.float()).sum() + (kk * gk.float()).sum()).backward()
    assert _rel(g_qb, ql.grad) < 6e-3
    assert _rel(g_kvb, kvl.grad) < 6e-3
    assert _rel(g_a[:, 8:8 + dr], krl.grad) < 6e-3
    assert (g_a[:, :8] == 0).all() and (g_a[:, 8 + dr:] == 0).all()
    assert _rel(ggq, qgl.grad) < 1e-3 and _rel(ggk, kgl.grad) < 1e-3


def test_outgate_situ_scale_add(R):
    from imfvideo_b200.ops import reference as ref

    torch.manual_seed(0)
    rows, hv, na = 333, 256, 528
    o, do = _rn(rows, hv, dt=BF16), _rn(rows, hv, dt=BF16)
    a, da = _rn(rows, na, dt=BF16), _rn(rows, na, dt=BF16)
    gcol = 272
    og, dog = torch.empty(rows, hv, dtype=BF16, device="cuda"), torch.empty(rows, hv, dtype=BF16, device="cuda")
    R.outgate_fwd(o, do, a[:, gcol:], da[:, gcol:], og, dog, rows, hv, hv, na)
    f = lambda x, z: x * torch.sigmoid(z)
    y0, dy0 = torch.func.jvp(f, (o.float(), a[:, gcol:].float()), (do.float(), da[:, gcol:].float()))
    assert _rel(og, y0) < 5e-3 and _rel(dog, dy0) < 5e-3
    gout = _rn(rows, hv, dt=BF16)
    g_o = torch.empty_like(o)
    g_a = torch.zeros_like(a)
    R.outgate_bwd(o, a[:, gcol:], gout, g_o, g_a[:, gcol:], rows, hv, hv, na, hv, na)
    ol, zl = o.float().requires_grad_(True), a[:, gcol:].float().requires_grad_(True)
    (f(ol, zl) * gout.float()).sum().backward()
    assert _rel(g_o, ol.grad) < 5e-3 and _rel(g_a[:, gcol:], zl.grad) < 5e-3
    # situ
    F_ = 688
    gu, dgu = _rn(rows, 2 * F_, dt=BF16, s=2.0), _rn(rows, 2 * F_, dt=BF16)
    act, dact = torch.empty(rows, F_, dtype=BF16, device="cuda"), torch.empty(rows, F_, dtype=BF16, device="cuda")
    for lb in (25.0, None):
        R.situ_fwd(gu, dgu, act, dact, rows, F_, 4.0, lb)
        y0, dy0 = ref.situ_mul_jvp(gu[:, :F_].float(), gu[:, F_:].float(), dgu[:, :F_].float(),
                                   dgu[:, F_:].float(), 4.0, lb)
        assert _rel(act, y0) < 5e-3 and _rel(dact, dy0) < 5e-3
        gact = _rn(rows, F_, dt=BF16)
        g_gu = torch.empty_like(gu)
        R.situ_bwd(gu, gact, g_gu, rows, F_, 4.0, lb)
        gl = gu.float().requires_grad_(True)
        (ref.situ_mul(gl[:, :F_], gl[:, F_:], 4.0, lb) * gact.float()).sum().backward()
        assert _rel(g_gu, gl.grad) < 6e-3
    # scale_add
    D = 256
    res, dres = _rn(rows, D), _rn(rows, D)
    y, dy = _rn(rows, D, dt=BF16), _rn(rows, D, dt=BF16)
    gate = _rn(D)
    out, dout = torch.empty(rows, D, device="cuda"), torch.empty(rows, D, device="cuda")
    R.scale_add_fwd(res, dres, y, dy, gate, out, dout, rows, D)
    assert _rel(out, res + y.float() * gate) < 1e-6 and _rel(dout, dres + dy.float() * gate) < 1e-6
    g = _rn(rows, D)
    g_y, g_gate = R.scale_add_bwd(y, gate, g, rows, D)
    assert _rel(g_y, g * gate) < 5e-3 and _rel(g_gate, (g * y.float()).sum(0)) < 1e-4
