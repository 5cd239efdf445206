"""CPU: SLA2 family -- routing, gather/state implementation vs dense fp32
reference, tangent, INT8 QAT, cube tiles with ragged prefix, model wiring
(model of the reference's tests/test_sla2_jvp.py, test_mla_video_sparse_jvp.py,
test_sla2_cube_qat.py, test_sla2_e2e.py)."""
import math
from functools import partial

import pytest
import torch

from imfvideo_b200.models import sla2 as S
from imfvideo_b200.models import IMFDiTVideo
from imfvideo_b200.ops.dual import Dual


def test_tile_permutation_round_trip():
    perm, inv, Np = S.tile_permutation((4, 4, 8), (2, 2, 4), prefix_len=5)
    L = 5 + 4 * 4 * 8
    x = torch.arange(L)
    assert Np == 8 and torch.equal(x[perm][inv], x)
    assert torch.equal(perm[-5:], torch.arange(5))          # prefix goes last
    first = perm[:16] - 5                                   # first tile: t<2, h<2, w<4
    t, h, w = first // 32, (first // 8) % 4, first % 8
    assert t.max() < 2 and h.max() < 2 and w.max() < 4


@pytest.mark.parametrize("L", [512, 640, 583])
def test_sparse_linear_matches_dense_and_tangent(L):
    torch.manual_seed(0)
    B, H, D, bq, bk = 1, 2, 16, 128, 64
    q, k, v, dq, dk, dv = (torch.randn(B, H, L, D) for _ in range(6))
    router = S.Router(D, bq, bk)
    with torch.no_grad():
        router.proj_q.weight.add_(0.1 * torch.randn(D, D))    # non-identity router
    mask, lut, topk, _ = router(q, k, 0.25)
    alpha = torch.rand(H, -(-L // bq))
    a_rows = alpha.repeat_interleave(bq, -1)[:, :L]
    f_fast = lambda a, b, c: S.sparse_linear_attention(a, b, c, lut, bq, bk, a_rows)
    f_ref = lambda a, b, c: S.sla2_dense(a, b, c, mask, alpha, bq, bk)
    o, do = torch.func.jvp(f_fast, (q, k, v), (dq, dk, dv))
    o0, do0 = torch.func.jvp(f_ref, (q, k, v), (dq, dk, dv))
    assert (o - o0).abs().max() < 2e-4 and (do - do0).abs().max() < 2e-3
    ql, kl, vl = (t.clone().requires_grad_(True) for t in (q, k, v))
    f_fast(ql, kl, vl).square().sum().backward()
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    f_ref(qr, kr, vr).square().sum().backward()
    for a, b in ((ql, qr), (kl, kr), (vl, vr)):
        assert (a.grad - b.grad).abs().max() < 2e-3


def test_soft_topk_rows_sum_to_budget_and_router_trains():
    torch.manual_seed(0)
    pc = torch.randn(2, 3, 5, 40)
    m = S.soft_topk(pc, 0.25)
    assert torch.allclose(m.sum(-1), torch.full((2, 3, 5), 10.0), atol=1e-2)
    mod = S.SLA2(16, topk=0.25, bq=64, bk=32)
    q, k, v = (torch.randn(1, 2, 256, 16) for _ in range(3))
    mod(q, k, v, soft_routing=True).square().sum().backward()
    assert mod.router.proj_q.weight.grad.abs().sum() > 0          # stage-1 router training


def test_cube_attention_matches_dense_reference_with_ragged_prefix():
    torch.manual_seed(0)
    grid, tile, P, H, D = (4, 4, 8), (2, 2, 4), 20, 2, 16
    L = P + 128
    impl = S.SLA2CubeQATAttentionImpl(D, L, H, grid, tile, topk=0.25, use_int8=False)
    assert impl.E == 16 and impl.Np == 8 and impl.n_tail == 2 and impl.Mb == 10
    with torch.no_grad():
        impl.alpha_logit.normal_()
        impl.proj_q.add_(0.1 * torch.randn(D, D))
    q, k, v, dq, dk, dv = (torch.randn(1, L, H, D) for _ in range(6))
    out = impl(Dual(q, dq), Dual(k, dk), Dual(v, dv))
    qh, kh, vh, dqh, dkh, dvh = (t[:, impl.perm].permute(0, 2, 1, 3) for t in (q, k, v, dq, dk, dv))
    lut_aug, T = impl.route(qh, kh)
    alpha = torch.sigmoid(impl.alpha_logit.detach())
    f = lambda a, b, c: S.cube_dense_ref(a, b, c, alpha, lut_aug[..., :T], impl.Np, impl.E, P)
    o0, do0 = torch.func.jvp(f, (qh, kh, vh), (dqh, dkh, dvh))
    back = lambda t: t.permute(0, 2, 1, 3)[:, impl.inv]
    assert (out.p - back(o0)).abs().max() < 2e-4
    assert (out.t - back(do0)).abs().max() < 2e-3


def test_int8_qat_close_to_float_and_has_gradients():
    torch.manual_seed(0)
    grid, tile, P, H, D = (4, 4, 8), (2, 2, 4), 20, 2, 16
    L = P + 128
    f32 = S.SLA2CubeQATAttentionImpl(D, L, H, grid, tile, topk=0.5, use_int8=False)
    i8 = S.SLA2CubeQATAttentionImpl(D, L, H, grid, tile, topk=0.5, use_int8=True)
    q, k, v = (torch.randn(1, L, H, D, requires_grad=True) for _ in range(3))
    o_f, o_q = f32(q, k, v), i8(q, k, v)
    assert (o_f - o_q).abs().max() < 5e-2 and not torch.equal(o_f, o_q)
    o_q.square().sum().backward()
    assert torch.isfinite(q.grad).all() and q.grad.abs().sum() > 0       # straight-through
    assert i8.alpha_logit.grad.abs().sum() > 0
    assert i8.logit_max_log2.shape == (H,) and torch.isfinite(i8.logit_max_log2).all()
    xq, xs = S.quantize_blocks(q.detach().permute(0, 2, 1, 3), 16)
    assert xq.dtype == torch.int8 and xq.abs().max() <= 127 and xs.shape == (1, H, math.ceil(L / 16))
    deq = S.fake_quant_blocks(q.detach().permute(0, 2, 1, 3), 16)
    assert torch.allclose(deq, (xq.float().view(1, H, -1, 16) * xs.repeat_interleave(16, -1)[..., :L, None]), atol=1e-6)


@pytest.mark.parametrize("kind", ["sla2_jvp", "sla2_cube_qat"])
def test_model_with_sla2_attention_state_dict_and_loss(kind):
    from imfvideo_b200.config import preset
    from imfvideo_b200.loss import IMFVideoLoss
    from imfvideo_b200.train import build_model

    cfg = preset("tiny")
    cfg.model.attn_impl = kind
    cfg.model.num_heads, cfg.model.qk_rope_head_dim = 2, 8
    cfg.model.sla2_topk, cfg.model.sla2_bq, cfg.model.sla2_bk = 0.25, 64, 32
    cfg.model.sla2_tile = (2, 2, 4)
    cfg.model.attn_res_block_size = 2
    net, _, _ = build_model(cfg)
    keys = set(net.state_dict().keys())
    if kind == "sla2_jvp":
        assert "shared_blocks.0.attn.attn_impl.sla2.router.proj_q.weight" in keys
        assert "shared_blocks.0.attn.attn_impl.sla2.alpha_logit" in keys
        assert not net.tile_major
    else:
        assert "shared_blocks.0.attn.attn_impl.proj_k" in keys
        assert "shared_blocks.0.attn.attn_impl.alpha_logit" in keys
        assert net.tile_major and "tm_perm" not in keys
    with torch.no_grad():
        for p in net.parameters():
            p.add_(0.03 * torch.randn_like(p))
    lm = IMFVideoLoss(net, 1000, data_proportion=0.25)
    x, y = torch.randn(2, 16, 4, 16, 16), torch.randint(0, 1000, (2,))
    loss, parts = lm(x, y)
    loss.backward()
    assert torch.isfinite(loss)
    grads = [p.grad for p in net.parameters() if p.grad is not None]
    assert all(torch.isfinite(g).all() for g in grads)
    alpha = [p.grad for n, p in net.named_parameters() if "alpha_logit" in n and p.grad is not None]
    assert alpha and any(a.abs().sum() > 0 for a in alpha)
