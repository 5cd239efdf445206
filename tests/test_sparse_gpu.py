"""GPU: block-sparse INT8 attention kernel (primal + tangent) and quantiser
against the SLA2 torch formulas."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def SP():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from imfvideo_b200.ops import cuda as cu

    assert cu.available()
    from imfvideo_b200.ops import sparse

    return sparse


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def test_quantiser_matches_reference(SP):
    from imfvideo_b200.models import sla2 as S

    torch.manual_seed(0)
    x = torch.randn(2, 333, 3, 64, device="cuda").bfloat16()
    xq, xs, xf = SP.quantize_blocks(x, 64, want_fq=True)
    rq, rs = S.quantize_blocks(x.permute(0, 2, 1, 3).float(), 64)
    diff = (xq.permute(0, 2, 1, 3).int() - rq.int()).abs()
    assert diff.max() <= 1 and (diff > 0).float().mean() < 1e-3
    assert torch.allclose(xs, rs, rtol=1e-6)
    rf = S.fake_quant_blocks(x.permute(0, 2, 1, 3).float(), 64).permute(0, 2, 1, 3)
    assert _rel(xf, rf) < 4e-3


def test_quantiser_of_three_tensors_in_one_launch(SP):
    """q, k, v of an attention call through one launch: bit-identical to three launches, with
    strided inputs (column views of a wider buffer) and with outputs left out per tensor."""
    torch.manual_seed(1)
    wide = torch.randn(2, 333, 3, 192, device="cuda").bfloat16()
    q, k, v = wide[..., :64], wide[..., 64:128], wide[..., 128:]
    many = SP.quantize_blocks_many([(q, True, False), (k, True, True), (v, False, True)])
    one = [SP.quantize_blocks(q, 64), SP.quantize_blocks(k, 64, want_fq=True),
           SP.quantize_blocks(v, 64, want_q=False, want_fq=True)]
    for (aq, as_, af), (bq, bs, bf) in zip(many, one):
        assert (aq is None) == (bq is None) and (af is None) == (bf is None)
        assert torch.equal(as_, bs)
        assert aq is None or torch.equal(aq, bq)
        assert af is None or torch.equal(af, bf)
    # differing shapes: one launch per tensor, same results
    q2 = torch.randn(2, 100, 3, 64, device="cuda").bfloat16()
    mixed = SP.quantize_blocks_many([(q2, True, False), (k, True, False)])
    assert torch.equal(mixed[0][0], SP.quantize_blocks(q2, 64)[0])
    assert torch.equal(mixed[1][0], one[1][0])


def test_tile_lut_union(SP):
    sel = torch.tensor([[[[0, 3], [3, 5], [1, 2]]]], device="cuda")        # Mb = 3, T = 2
    lut, fl = SP.build_tile_lut(sel, 64)
    assert lut.shape == (1, 1, 2, 4)
    assert lut[0, 0, 0].tolist() == [0, 3, 5, -1] and fl[0, 0, 0].tolist()[:3] == [1, 3, 2]
    assert lut[0, 0, 1].tolist() == [1, 2, -1, -1] and fl[0, 0, 1].tolist()[:2] == [1, 1]


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("qblk,L", [(128, 640), (64, 583), (64, 1024)])
def test_sparse_forward_and_tangent(SP, int8, qblk, L):
    from imfvideo_b200.models import sla2 as S

    torch.manual_seed(L + qblk)
    B, H, D = 1, 2, 64
    mk = lambda s=1.0: (torch.randn(B, L, H, D, device="cuda") * s).bfloat16()
    q, k, v, dq, dk, dv = mk(), mk(), mk(), mk(.5), mk(.5), mk(.5)
    Mb, Nb = -(-L // qblk), -(-L // 64)
    T = max(2, Nb // 4)
    sel = torch.stack([torch.stack([torch.randperm(Nb, device="cuda")[:T] for _ in range(Mb)])
                       for _ in range(H)]).unsqueeze(0)
    lut, flags = SP.build_tile_lut(sel, qblk)
    o, do, lse = SP.sparse_fwd(q, k, v, dq, dk, dv, lut, flags, qblk, int8, quant_p=int8)
    o2, _, _ = SP.sparse_fwd(q, k, v, None, None, None, lut, flags, qblk, int8, quant_p=int8)
    ph = lambda t: t.permute(0, 2, 1, 3).float()
    a_rows = torch.ones(H, L, device="cuda")          # alpha = 1: sparse branch only

    def f(a, b, c):
        out, o_s, _o_l, ls = S.sparse_linear_attention(a, b, c, sel, qblk, 64, a_rows, int8=int8,
                                                       return_parts=True)
        return o_s, ls
    (ro, rl), (rdo, _) = torch.func.jvp(f, (ph(q), ph(k), ph(v)), (ph(dq), ph(dk), ph(dv)))
    tol = 3e-2 if int8 else 1e-2
    assert _rel(o.permute(0, 2, 1, 3), ro) < tol
    assert _rel(do.permute(0, 2, 1, 3), rdo) < (8e-2 if int8 else 1.5e-2)
    assert (lse - rl).abs().max() < (5e-2 if int8 else 2e-3)
    assert _rel(o2, o) < 5e-3
    from imfvideo_b200.ops import kernels
    kernels.check_status()


@pytest.mark.parametrize("kind", ["sla2_jvp", "sla2_cube_qat"])
def test_sla2_model_fused_core_vs_torch_formulas(SP, kind):
    """Model with SLA2 attention: fused block node + sparse kernel vs the op-by-op
    torch path (same routing, same INT8 grid)."""
    from imfvideo_b200.config import preset
    from imfvideo_b200.ops import cuda as cu
    from imfvideo_b200.ops import kernels
    from imfvideo_b200.ops.dual import Dual
    from imfvideo_b200.train import build_model

    cfg = preset("d256")
    cfg.model.depth, cfg.model.aux_head_depth = 2, 1
    cfg.model.attn_impl = kind
    cfg.model.sla2_topk, cfg.model.sla2_bq, cfg.model.sla2_bk = 0.25, 128, 64
    cfg.model.sla2_tile = (4, 4, 4)
    cfg.data.latent_frames, cfg.data.latent_size = 8, (16, 32)      # grid (8, 8, 16) -> 16 tiles
    torch.manual_seed(0)
    net, _, _ = build_model(cfg)
    net = net.cuda()
    net.compute_dtype = torch.bfloat16
    with torch.no_grad():
        for p in net.parameters():
            p.add_(torch.randn_like(p) * 0.03)
    B = 1
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(B, 16, 8, 16, 32, device="cuda", generator=g)
    dx = torch.randn(B, 16, 8, 16, 32, device="cuda", generator=g)
    h = torch.rand(B, device="cuda", generator=g)
    w = 1 + torch.rand(B, device="cuda", generator=g)
    lo, hi = torch.zeros(B, device="cuda"), torch.ones(B, device="cuda")
    y = torch.randint(0, 1000, (B,), device="cuda")

    def run():
        net.zero_grad()
        out = net.forward_dual(Dual(x, dx), Dual(h, torch.ones_like(h)), w, lo, hi, y)
        (out["u"].p.square().sum() + out["v"].p.square().sum()).backward()
        return out, {n: p.grad.clone() for n, p in net.named_parameters() if p.grad is not None}

    n0 = kernels.LAUNCHES.count
    out_f, g_f = run()
    kernels.check_status()
    assert kernels.LAUNCHES.count - n0 > 20
    cu.disable("block")
    try:
        out_g, g_g = run()
    finally:
        cu.enable("block")
    assert _rel(out_f["u"].p, out_g["u"].p) < 5e-2 and _rel(out_f["v"].p, out_g["v"].p) < 5e-2
    assert _rel(out_f["u"].t, out_g["u"].t) < 8e-2
    al = [n for n in g_f if "alpha_logit" in n]
    assert al and all(torch.isfinite(g_f[n]).all() for n in g_f)
    bad = [(n, _rel(g_f[n], g_g[n])) for n in g_g if n in g_f and g_g[n].norm() > 0
           and _rel(g_f[n], g_g[n]) > 0.15]
    # The only gradients that leave the 15 % band are gains of the attention-residual score
    # heads (``*_res_norm.weight``): their gradient is the small difference of large
    # per-candidate terms of a softmax over 2-3 candidates, so the bf16 rounding of the mixed
    # stream shows up in it (17 % on one such gain with the 1-D SLA2 blocks, none with cubes).
    assert all("_res_norm" in n and r < 0.25 for n, r in bad) and len(bad) <= 1, bad


@pytest.mark.parametrize("qblk,L", [(128, 640), (64, 583)])
def test_sparse_backward_kernel(SP, qblk, L):
    from imfvideo_b200.models import sla2 as S
    from imfvideo_b200.ops import kernels

    torch.manual_seed(L)
    B, H, D = 1, 2, 64
    mk = lambda: torch.randn(B, L, H, D, device="cuda").bfloat16()
    q, k, v, go = mk(), mk(), mk(), mk()
    Mb, Nb = -(-L // qblk), -(-L // 64)
    T = max(2, Nb // 4)
    sel = torch.stack([torch.stack([torch.randperm(Nb, device="cuda")[:T] for _ in range(Mb)])
                       for _ in range(H)]).unsqueeze(0)
    lut, flags = SP.build_tile_lut(sel, qblk)
    o, _, lse = SP.sparse_fwd(q, k, v, None, None, None, lut, flags, qblk, False, quant_p=False)
    qlist, qflags = SP.build_kv_lists(lut, flags, L)
    dq, dk, dv = kernels.attn_bwd(q, k, v, o, lse, go, qlist=qlist, qflags=qflags)
    ph = lambda t: t.permute(0, 2, 1, 3).float()
    ql, kl, vl = (ph(t).requires_grad_(True) for t in (q, k, v))
    a_rows = torch.ones(H, L, device="cuda")
    _, o_s, _, _ = S.sparse_linear_attention(ql, kl, vl, sel, qblk, 64, a_rows, return_parts=True)
    o_s.backward(ph(go))
    for name, a, b in (("dq", dq, ql.grad), ("dk", dk, kl.grad), ("dv", dv, vl.grad)):
        assert _rel(a.permute(0, 2, 1, 3), b) < 2e-2, (name, _rel(a.permute(0, 2, 1, 3), b))
    kernels.check_status()


def test_sparse_backward_bitwise_repeatable(SP):
    from imfvideo_b200.ops import kernels
    """Block-sparse backward with the device-built lists and ranks: dQ bit-identical from run
    to run (fixed order of additions), and equal to the arrival-order result up to rounding."""
    torch.manual_seed(11)
    B, H, L, qblk = 1, 3, 5000, 64
    mk = lambda: torch.randn(B, L, H, 64, device="cuda").bfloat16()
    q, k, v, go = mk(), mk(), mk(), mk()
    Mb, Nb = -(-L // qblk), -(-L // 64)
    T = max(2, Nb // 5)
    sel = torch.stack([torch.stack([torch.randperm(Nb, device="cuda")[:T] for _ in range(Mb)])
                       for _ in range(H)]).unsqueeze(0).int()
    lut, flags, cnt, maps = SP.route_tables(sel, qblk, L)
    o, _, lse = SP.sparse_fwd(q, k, v, None, None, None, lut, flags, qblk, False, quant_p=False,
                              cnt=cnt)
    qlist, qflags, qrank = SP.kv_lists(maps, want_rank=True)
    kernels.set_deterministic(True)
    try:
        first = kernels.attn_bwd(q, k, v, o, lse, go, qlist=qlist, qflags=qflags, qrank=qrank)
        for _ in range(3):
            again = kernels.attn_bwd(q, k, v, o, lse, go, qlist=qlist, qflags=qflags, qrank=qrank)
            assert all(torch.equal(a, b) for a, b in zip(first, again))
    finally:
        kernels.set_deterministic(False)
    loose = kernels.attn_bwd(q, k, v, o, lse, go, qlist=qlist, qflags=qflags)   # arrival order
    assert _rel(loose[0], first[0]) < 1e-3
    assert torch.equal(loose[1], first[1]) and torch.equal(loose[2], first[2])
    kernels.check_status()


def test_linear_branch_kernels_match_formulas():
    """Complement linear branch (states, mask product on the tcgen05 GEMM, apply, reverse
    mode) against the fp32 formulas of models/sla2.py and their torch.func.jvp / autograd."""
    from imfvideo_b200.models.sla2 import linear_branch
    from imfvideo_b200.ops import linattn as LA

    assert LA.AVAILABLE
    torch.manual_seed(3)
    dev = "cuda"
    B, L, H, D, blk, T, n_comp = 2, 1000, 2, 64, 64, 3, 14
    Mb = Nb = -(-L // blk)
    mk = lambda: torch.randn(B, L, H, D, device=dev).bfloat16()
    q, k, v, dq, dk, dv, o_s, do_s, go = (mk() for _ in range(9))
    sel = torch.stack([torch.stack([torch.stack([torch.randperm(Nb, device=dev)[:T]
                                                 for _ in range(Mb)]) for _ in range(H)])
                       for _ in range(B)]).int()
    logit = torch.randn(H, L, device=dev, requires_grad=True)
    hp = lambda t: t.permute(0, 2, 1, 3).float()
    f = lambda a, b, c: linear_branch(a, b, c, sel, blk, blk, n_comp)
    o_l, do_l = torch.func.jvp(f, (hp(q), hp(k), hp(v)), (hp(dq), hp(dk), hp(dv)))
    a4 = torch.sigmoid(logit).detach().t().reshape(1, L, H, 1)
    o_ref = a4 * o_s.float() + (1 - a4) * o_l.permute(0, 2, 1, 3)
    do_ref = a4 * do_s.float() + (1 - a4) * do_l.permute(0, 2, 1, 3)
    a_rows = torch.sigmoid(logit).detach()
    o, do, C = LA.forward(q, k, v, dq, dk, dv, o_s, do_s, sel, a_rows, blk, blk, n_comp)
    rel = lambda x, y: ((x.float() - y.float()).norm() / y.float().norm()).item()
    assert rel(o, o_ref) < 6e-3 and rel(do, do_ref) < 6e-3
    o1, _, _ = LA.forward(q, k, v, None, None, None, o_s, None, sel, a_rows, blk, blk, n_comp)
    assert torch.equal(o1, o)
    # reverse mode
    ql, kl, vl = (hp(t).requires_grad_(True) for t in (q, k, v))
    al = torch.sigmoid(logit).t().reshape(1, L, H, 1)
    mix = al * o_s.float() + (1 - al) * linear_branch(ql, kl, vl, sel, blk, blk, n_comp).permute(0, 2, 1, 3)
    gq_r, gk_r, gv_r, gl_r = torch.autograd.grad(mix, (ql, kl, vl, logit), go.float())
    gq_l, gnum, gden, ga_row, g_os = LA.backward_rows(q, o_s, go, C, a_rows, blk)
    assert rel(gq_l, gq_r.permute(0, 2, 1, 3)) < 2e-3
    assert rel(ga_row.sum(0), gl_r) < 2e-3
    assert rel(g_os, a4 * go.float()) < 6e-3
    zero = torch.zeros_like(q)
    gk, gv = LA.backward_kv(q, k, v, gnum, gden, sel, zero, zero, blk, blk, n_comp)
    assert rel(gk, gk_r.permute(0, 2, 1, 3)) < 6e-3
    assert rel(gv, gv_r.permute(0, 2, 1, 3)) < 6e-3


@pytest.mark.parametrize("qblk", [64, 128])
def test_device_routing_tables_match_torch_builders(SP, qblk):
    torch.manual_seed(5)
    dev = "cuda"
    B, H, L, T = 2, 3, 1500, 5
    Mb, Nb = -(-L // qblk), -(-L // 64)
    sel = torch.stack([torch.stack([torch.stack([torch.randperm(Nb, device=dev)[:T]
                                                 for _ in range(Mb)]) for _ in range(H)])
                       for _ in range(B)]).int()
    lut_r, fl_r = SP.build_tile_lut(sel, qblk)
    lut, fl, cnt, fm = SP.route_tables(sel, qblk, L)
    if qblk == 128:     # the torch builder keeps the selection order, the kernel sorts
        order = lut_r.sort(-1).indices
        lut_r, fl_r = torch.gather(lut_r, -1, order), torch.gather(fl_r, -1, order)
    n = lut_r.shape[-1]
    assert torch.equal(cnt, (lut_r >= 0).sum(-1).int())
    big = torch.iinfo(torch.int32).max
    key = lambda t: torch.where(t < 0, torch.full_like(t, big), t).sort(-1).values
    assert torch.equal(key(lut[..., :n]), key(lut_r))
    valid = lut[..., :n] >= 0
    if qblk == 64:
        assert torch.equal(lut[..., :n][valid], lut_r[lut_r >= 0])
        assert torch.equal(fl[..., :n][valid], fl_r[lut_r >= 0])
    ql_r, qf_r = SP.build_kv_lists(lut_r, fl_r, L)
    ql, qf, qr = SP.kv_lists(fm, want_rank=True)
    m = ql_r.shape[-1]
    assert bool((ql[..., m:] < 0).all())
    assert torch.equal(ql[..., :m], ql_r) and torch.equal(qf[..., :m], qf_r)
    # rank of an entry = how many higher K/V tiles attend the same query tile
    live = fm[2] != 0                                           # (B, H, n_kvt, n_mt)
    above = live.flip(2).cumsum(2).flip(2) - live.long()
    valid = ql >= 0
    want = torch.gather(above, 3, ql.clamp(min=0).long())
    assert torch.equal(qr.long()[valid], want[valid])


@pytest.mark.parametrize("L,bq,bk,n_keys,n_tail,proj", [
    (29140, 64, 64, 455, 1, True),        # cube shape: 455 video tiles + 1 prefix tail block
    (1000, 128, 64, None, 0, True),       # 1-D router, ragged last blocks
    (700, 64, 64, None, 0, False),
])
def test_router_pool_and_topk_kernels(SP, L, bq, bk, n_keys, n_tail, proj):
    """Pooled block means and the radix-select top-k against torch: the means and scores
    match the fp32 formulas; the selection is an exact top-T of the kernel's own scores
    (so a rounding-level difference of two near-equal scores cannot fail the test)."""
    from imfvideo_b200.models import sla2 as S

    torch.manual_seed(5)
    B, H = 2, 3
    q = torch.randn(B, L, H, 64, device="cuda").bfloat16().permute(0, 2, 1, 3)
    k = torch.randn(B, L, H, 64, device="cuda").bfloat16().permute(0, 2, 1, 3)
    qb = SP.pool_blocks(q, bq)
    nkb = n_keys if n_keys is not None else -(-L // bk)
    kb = SP.pool_blocks(k, bk, nkb)
    assert torch.allclose(qb, S.block_mean(q, bq), atol=1e-5)
    assert torch.allclose(kb, S.block_mean(k, bk)[:, :, :nkb], atol=1e-5)
    pq = pk = None
    if proj:
        pq = torch.eye(64, device="cuda") + 0.3 * torch.randn(64, 64, device="cuda")
        pk = torch.eye(64, device="cuda") + 0.3 * torch.randn(64, 64, device="cuda")
    T = max(1, int(0.05 * nkb))
    sel, sc = SP.route_topk(qb, kb, T, pq, pk, n_tail=n_tail, tail0=nkb, want_scores=True)
    qp = qb if pq is None else qb @ pq.t()
    kp = kb if pk is None else kb @ pk.t()
    ref = (qp @ kp.transpose(-1, -2)) * 64 ** -0.5
    assert torch.allclose(sc, ref, atol=2e-5, rtol=1e-4)
    top = sel[..., :T].long()
    assert int(top.min()) >= 0 and int(top.max()) < nkb
    assert bool((top[..., 1:] != top[..., :-1]).all())
    picked = torch.zeros_like(sc, dtype=torch.bool).scatter_(-1, top, True)
    assert int(picked.sum(-1).min()) == T                       # no duplicates
    lo_in = sc.masked_fill(~picked, float("inf")).amin(-1)
    hi_out = sc.masked_fill(picked, float("-inf")).amax(-1)
    assert bool((lo_in >= hi_out).all())
    want = torch.topk(sc, T, dim=-1).indices.sort(-1).values
    assert (top.sort(-1).values == want).float().mean() > 0.999
    if n_tail:
        assert bool((sel[..., T:] == torch.arange(nkb, nkb + n_tail, device="cuda")).all())


def test_router_modules_use_the_kernels(SP):
    """Router.forward (1-D) and route_tiles (cube) on the kernels agree with their torch paths."""
    from imfvideo_b200.models import sla2 as S

    torch.manual_seed(6)
    B, H, L = 1, 2, 64 * 40 + 20
    q = torch.randn(B, L, H, 64, device="cuda").bfloat16().permute(0, 2, 1, 3)
    k = torch.randn(B, L, H, 64, device="cuda").bfloat16().permute(0, 2, 1, 3)
    r = S.Router(64, bq=128, bk=64).cuda()
    with torch.no_grad():
        r.proj_q.weight.add_(0.2 * torch.randn_like(r.proj_q.weight))
    _, lut_k, tk, _ = r(q, k, 0.1, need_mask=False)
    _, lut_t, tt, _ = r(q.float(), k.float(), 0.1, need_mask=False)
    assert tk == tt and lut_k.shape == lut_t.shape
    same = (lut_k.sort(-1).values == lut_t.sort(-1).values.to(lut_k.dtype)).float().mean()
    assert same > 0.99
    lut_c, T = S.route_tiles(q, k, 0.1, 40, 64, 20, n_tail=1)
    lut_r, T2 = S.route_tiles(q.float(), k.float(), 0.1, 40, 64, 20, n_tail=1)
    assert T == T2 and lut_c.shape == lut_r.shape == (B, H, 41, T + 1)
    same = (lut_c.sort(-1).values == lut_r.sort(-1).values.to(lut_c.dtype)).float().mean()
    assert same > 0.99


def test_complement_mask_kernel_matches_scatter(SP):
    from imfvideo_b200.ops import linattn as LA

    torch.manual_seed(7)
    B, H, Mb, Nb, T = 2, 3, 37, 41, 6
    sel = torch.stack([torch.randperm(Nb, device="cuda")[:T] for _ in range(B * H * Mb)])
    sel = sel.view(B, H, Mb, T).to(torch.int32)
    for transpose in (False, True):
        got = LA.comp_mask(sel, Mb, Nb, transpose)
        cm = torch.ones(B, H, Mb, Nb, device="cuda").scatter_(-1, sel.long(), 0.0)
        if transpose:
            cm = cm.transpose(-1, -2)
        rows, cols = cm.shape[-2:]
        cp = (cols + 3) // 4 * 4
        want = torch.zeros(B * H, rows, 2 * cp, device="cuda")
        want[:, :, :cols] = cm.reshape(B * H, rows, cols)
        want[:, :, cp:cp + cols] = cm.reshape(B * H, rows, cols)
        assert got.dtype == torch.bfloat16 and torch.equal(got.float(), want)


def test_sla2_sampler_kernels_vs_torch_formulas(SP):
    """The few-step sampler of an SLA2 cube model (no-grad, primal-only kernels, INT8 score
    grid) against the op-by-op torch path with the same routing: within the QAT tolerance."""
    from imfvideo_b200.config import preset
    from imfvideo_b200.loss import IMFVideoLoss
    from imfvideo_b200.ops import cuda as cu
    from imfvideo_b200.ops import kernels
    from imfvideo_b200.train import build_model

    cfg = preset("d256_sla2")
    cfg.model.depth, cfg.model.aux_head_depth = 3, 1
    cfg.model.sla2_topk = 0.25
    cfg.data.latent_frames, cfg.data.latent_size = 8, (16, 32)
    torch.manual_seed(0)
    net, _, _ = build_model(cfg)
    net = net.cuda().eval()
    net.compute_dtype = torch.bfloat16
    with torch.no_grad():
        for p in net.parameters():
            p.add_(torch.randn_like(p) * 0.03)
    loss = IMFVideoLoss(net, cfg.model.num_classes, autocast_bf16=True)
    g = torch.Generator(device="cuda").manual_seed(2)
    z = torch.randn(1, 16, 8, 16, 32, device="cuda", generator=g)
    y = torch.randint(0, 1000, (1,), device="cuda")
    n0 = kernels.LAUNCHES.count
    out_k = loss.sample(z, y, num_steps=4)
    kernels.check_status()
    assert kernels.LAUNCHES.count - n0 > 50
    cu.disable("block")
    try:
        out_t = loss.sample(z, y, num_steps=4)
    finally:
        cu.enable("block")
    assert torch.isfinite(out_k).all()
    assert _rel(out_k, out_t) < 5e-2
