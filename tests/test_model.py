"""CPU: model semantics -- dual-number pass vs torch.func.jvp, gradient
parity with the plain forward, state_dict parity with the reference model,
loss / sampler plumbing (model of the reference's tests/test_model_pt.py)."""
import copy

import pytest
import torch

from imfvideo_b200.loss import IMFVideoLoss
from imfvideo_b200.models import IMFDiTVideo
from imfvideo_b200.ops.dual import Dual

KW = dict(input_size=16, num_frames=4, hidden_size=64, depth=3, num_heads=2, aux_head_depth=1,
          kv_lora_rank=32, qk_rope_head_dim=16, mlp_ratio=4.0)


def _net(**over):
    torch.manual_seed(0)
    net = IMFDiTVideo(**{**KW, **over})
    with torch.no_grad():      # zero-init gates / final layers would make du/dt == 0
        for p in net.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    return net


def _inputs(B=2):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(B, 16, 4, 16, 16, generator=g)
    dx = torch.randn(B, 16, 4, 16, 16, generator=g)
    t = torch.rand(B, generator=g)
    r = torch.rand(B, generator=g) * t
    w = 1 + 3 * torch.rand(B, generator=g)
    lo, hi = 0.5 * torch.rand(B, generator=g), 0.5 + 0.5 * torch.rand(B, generator=g)
    y = torch.randint(0, 1000, (B,), generator=g)
    return x, dx, t, r, w, lo, hi, y


@pytest.mark.parametrize("bs", [0, 2])
@pytest.mark.parametrize("ckpt", [False, True])
def test_dual_pass_matches_functorch(bs, ckpt):
    net = _net(attn_res_block_size=bs, grad_checkpoint=ckpt)
    x, dx, t, r, w, lo, hi, y = _inputs()
    fn = lambda z, tt, rr: net(z, tt, tt - rr, w, lo, hi, y)
    u0, du0, v0 = torch.func.jvp(fn, (x, t, r), (dx, torch.ones_like(t), torch.zeros_like(t)),
                                 has_aux=True)
    out = net.forward_dual(Dual(x, dx), Dual(t - r, torch.ones_like(t)), w, lo, hi, y)
    assert du0.abs().max() > 1e-3
    assert torch.allclose(out["u"].p, u0, atol=1e-5)
    assert torch.allclose(out["u"].t, du0, atol=2e-4)
    assert torch.allclose(out["v"].p, v0, atol=1e-5) and out["v"].t is None
    # reverse mode through the dual pass == reverse mode through the plain forward
    net.zero_grad()
    (out["u"].p.square().sum() + out["v"].p.sum()).backward()
    g1 = {n: p.grad.clone() for n, p in net.named_parameters() if p.grad is not None}
    net.zero_grad()
    uu, vv = net(x, t, t - r, w, lo, hi, y)
    (uu.square().sum() + vv.sum()).backward()
    for n, p in net.named_parameters():
        if p.grad is not None:
            assert torch.allclose(g1[n], p.grad, atol=1e-5), n


def test_branch_selection_and_eval_mode():
    net = _net()
    x, dx, t, r, w, lo, hi, y = _inputs()
    full = net.forward_dual(Dual(x), Dual(t - r), w, lo, hi, y)
    only_v = net.forward_dual(Dual(x), Dual(t - r), w, lo, hi, y, branches=("v",))
    assert set(only_v) == {"v"} and torch.equal(only_v["v"].p, full["v"].p)
    ev = _net(eval_mode=True)
    u, v = ev(x, t, t - r, w, lo, hi, y)
    assert len(ev.v_heads) == 0 and torch.equal(u, v)


def test_mla_geometry_defaults():
    net = IMFDiTVideo(input_size=(8, 16), num_frames=2, hidden_size=256, depth=2, num_heads=4,
                      aux_head_depth=1)
    a = net.shared_blocks[0].attn
    assert (a.qk_nope_head_dim, a.qk_rope_head_dim, a.v_head_dim) == (48, 16, 64)
    assert (a.q_lora_rank, a.kv_lora_rank) == (128, 64)
    assert net.prefix_tokens == 20 and net.seq_len == 20 + 2 * 4 * 8
    assert net.rope_cos.shape == (net.seq_len, 8)
    assert "rope_cos" not in net.state_dict()


@pytest.mark.parametrize("bs", [0, 2])
def test_state_dict_and_forward_parity_with_reference(ref_modules, bs):
    R = ref_modules["models.imf_dit_video"]
    kw = dict(KW, attn_res_block_size=bs)
    torch.manual_seed(0)
    theirs = R.IMFDiTVideo(**kw)
    ours = IMFDiTVideo(**kw)
    sd_t, sd_o = theirs.state_dict(), ours.state_dict()
    assert list(sd_t.keys()) == list(sd_o.keys())
    assert all(sd_t[k].shape == sd_o[k].shape for k in sd_t)
    with torch.no_grad():
        for p in theirs.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    ours.load_state_dict(theirs.state_dict())
    x, dx, t, r, w, lo, hi, y = _inputs()
    u_t, v_t = theirs(x, t, t - r, w, lo, hi, y)
    u_o, v_o = ours(x, t, t - r, w, lo, hi, y)
    assert torch.allclose(u_o, u_t, atol=2e-5) and torch.allclose(v_o, v_t, atol=2e-5)


def test_loss_matches_reference_loss(ref_modules):
    """Same seed -> same sampled (t, r, omega, ...) -> same loss value."""
    net = _net()
    ours = IMFVideoLoss(net, 1000, data_proportion=0.25, jvp_impl="fused")
    theirs = ref_modules["imf_video"].IMFVideoLoss(net, 1000, data_proportion=0.25,
                                                  jvp_impl="functorch")
    x, _, _, _, _, _, _, y = _inputs(4)
    torch.manual_seed(7)
    l_o, d_o = ours(x, y)
    torch.manual_seed(7)
    l_t, d_t = theirs(x, y)
    assert torch.allclose(l_o, l_t, atol=1e-5)
    assert torch.allclose(d_o["loss_u"], d_t["loss_u"], rtol=1e-4)


@pytest.mark.parametrize("impl", ["fused", "functorch"])
def test_loss_backward_finite_and_sampler(impl):
    net = _net(attn_res_block_size=2)
    lm = IMFVideoLoss(net, 1000, data_proportion=0.25, jvp_impl=impl)
    x, _, _, _, _, _, _, y = _inputs(4)
    loss, parts = lm(x, y)
    loss.backward()
    assert torch.isfinite(loss) and all(torch.isfinite(v) for v in parts.values())
    grads = [p.grad for p in net.parameters() if p.grad is not None]
    assert grads and all(torch.isfinite(g).all() for g in grads)
    for steps in (1, 4):
        z = lm.sample(torch.randn(2, 16, 4, 16, 16), y[:2], num_steps=steps, omega=2.0)
        assert z.shape == (2, 16, 4, 16, 16) and torch.isfinite(z).all()


def test_reuse_ungated_guidance_is_exact():
    net = _net()
    x, _, _, _, _, _, _, y = _inputs(6)
    a = IMFVideoLoss(net, 1000, data_proportion=0.25)
    b = IMFVideoLoss(net, 1000, data_proportion=0.25, reuse_ungated_guidance=True)
    torch.manual_seed(3)
    la, _ = a(x, y)
    torch.manual_seed(3)
    lb, _ = b(x, y)
    assert torch.allclose(la, lb, atol=1e-6)


def test_sampling_laws():
    lm = IMFVideoLoss(_net(), 1000, data_proportion=0.25, strat_group=8)
    t, r, fm = lm.sample_tr(64, "cpu", torch.float32)
    assert (r <= t).all() and (r[fm] == t[fm]).all()
    assert abs(fm.float().mean().item() - 0.25) < 0.05          # stratified split
    om = lm.sample_cfg_scale(64, "cpu")
    assert om.min() >= 1.0 and om.max() <= 8.0 + 1e-4
    lo, hi = lm.sample_cfg_interval(64, "cpu", torch.float32, fm)
    assert (lo[fm] == 0).all() and (hi[fm] == 1).all() and (lo <= 0.5).all() and (hi >= 0.5).all()
    # cross-micro-batch strata: 8 single draws cover all 8 strata exactly once
    lm2 = IMFVideoLoss(_net(), 1000, strat_group=8)
    us = torch.cat([lm2._strat_uniform(1, "cpu", "s") for _ in range(8)])
    assert sorted((us * 8).floor().int().tolist()) == list(range(8))


def test_layout_formulas_are_adjoint_and_match_conv3d():
    """CPU path of the layout ops: patch rows x flattened Conv3d weight equals the
    convolution, scatter inverts gather in both feature orders, gather / scatter are
    adjoint (the autograd rules of the CUDA kernels rely on it), and a row permutation
    falls back to plain indexing."""
    from imfvideo_b200.ops import patch as PK

    torch.manual_seed(0)
    B, C, T, H, W, patch = 2, 4, 4, 6, 8, (2, 2, 2)
    x = torch.randn(B, C, T, H, W)
    conv = torch.nn.Conv3d(C, 10, kernel_size=patch, stride=patch)
    rows = PK.patch_rows(x, patch, c_last=False)
    y = rows @ conv.weight.reshape(10, -1).t() + conv.bias
    ref = conv(x).flatten(2).transpose(1, 2)
    assert torch.allclose(y, ref, atol=1e-5)
    for c_last in (False, True):
        r = PK.patch_rows(x, patch, c_last)
        assert torch.equal(PK.unpatch_rows(r, x.shape, patch, c_last), x)
        g = torch.randn_like(r)
        lhs = (r * g).sum()
        rhs = (x * PK.scatter_formula(g, x.shape, patch, c_last)).sum()
        assert torch.allclose(lhs, rhs, rtol=1e-5)
    z = torch.randn(2, 12, 8)
    perm = torch.randperm(12)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(12)
    assert torch.equal(PK.permute_rows(z, perm, inv), z[:, perm])
    assert torch.equal(PK.permute_rows(PK.permute_rows(z, perm, inv), inv, perm), z)


def test_reference_import_names_and_fast_engine():
    """The reference's module paths resolve, plug-ins accept plain tensors, and
    ``model_du_dt_fast`` equals ``torch.func.jvp`` of the u output."""
    import importlib

    for mod, names in {"models.attention_op": ["flash_jvp_attention"],
                       "models.mla_jvp_fast": ["build_fast_jvp_state", "model_du_dt_fast"],
                       "models.sla2_attention": ["SLA2AttentionImpl"],
                       "models.sla2_cube_qat": ["SLA2CubeQATAttentionImpl"],
                       "models.imf_dit_video": ["eager_math_attention", "IMFDiTVideo"]}.items():
        m = importlib.import_module(mod)
        assert all(hasattr(m, n) for n in names), mod
    from models.attention_op import flash_jvp_attention
    from models.mla_jvp_fast import build_fast_jvp_state, model_du_dt_fast

    q, k, v = (torch.randn(1, 20, 2, 16) for _ in range(3))
    o = flash_jvp_attention(q, k, v)
    assert torch.is_tensor(o) and o.shape == (1, 20, 2, 16)
    net = _net(attn_res_block_size=1)
    b = 2
    x, v_c = torch.randn(b, 16, 4, 16, 16), torch.randn(b, 16, 4, 16, 16)
    t, r = torch.rand(b) * 0.5 + 0.5, torch.rand(b) * 0.5
    w, t0, t1 = torch.ones(b) * 1.5, torch.zeros(b), torch.ones(b)
    y = torch.randint(0, 1000, (b,))
    du = model_du_dt_fast(net, build_fast_jvp_state(net), x, t, t - r, w, t0, t1, y, v_c)
    fn = lambda z, tt: net(z, tt, tt - r, w, t0, t1, y)[0]
    _, want = torch.func.jvp(fn, (x, t), (v_c, torch.ones_like(t)))
    assert (du - want).abs().max() < 1e-4 * max(1.0, want.abs().max().item())
