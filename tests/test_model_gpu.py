"""GPU: the model / trainer through the kernel library vs the torch path."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kernels():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from imfvideo_b200.ops import cuda as cu

    assert cu.available()
    from imfvideo_b200.ops import kernels as K

    return K


def _net(dtype=None, bs=2, wide=False):
    """``wide``: 3 heads of 128 (not a power of two, the Wan2.1-1.3B head shape) and an MLP
    width that is not a multiple of 128."""
    from imfvideo_b200.models import IMFDiTVideo, flash_jvp_attention

    torch.manual_seed(0)
    geo = dict(hidden_size=384, num_heads=3, mlp_ratio=8960 / 1536) if wide else \
        dict(hidden_size=256, num_heads=4, kv_lora_rank=128)
    net = IMFDiTVideo(input_size=(16, 32), num_frames=4, depth=3, aux_head_depth=1,
                      attn_res_block_size=bs, attn_impl=flash_jvp_attention, compute_dtype=dtype,
                      **geo)
    with torch.no_grad():
        for p in net.parameters():
            p.add_(torch.randn_like(p) * 0.03)
    return net.cuda()


def test_model_dual_pass_bf16_kernels_vs_fp32_torch(kernels):
    from imfvideo_b200.ops import cuda as cu
    from imfvideo_b200.ops.dual import Dual

    net = _net(torch.bfloat16)
    B = 2
    x, dx = torch.randn(B, 16, 4, 16, 32, device="cuda"), torch.randn(B, 16, 4, 16, 32, device="cuda")
    h = torch.rand(B, device="cuda")
    w = 1 + torch.rand(B, device="cuda")
    lo, hi = torch.zeros(B, device="cuda"), torch.ones(B, device="cuda")
    y = torch.randint(0, 1000, (B,), device="cuda")
    n0 = kernels.LAUNCHES.count
    out = net.forward_dual(Dual(x, dx), Dual(h, torch.ones_like(h)), w, lo, hi, y)
    assert kernels.LAUNCHES.count > n0
    kernels.check_status()
    net.compute_dtype = None
    cu.disable("gemm", "attention", "block")
    try:
        ref = net.forward_dual(Dual(x, dx), Dual(h, torch.ones_like(h)), w, lo, hi, y)
    finally:
        cu.enable("gemm", "attention", "block")
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()
    assert rel(out["u"].p, ref["u"].p) < 3e-2
    assert rel(out["u"].t, ref["u"].t) < 5e-2
    assert rel(out["v"].p, ref["v"].p) < 3e-2


def test_trainer_steps_on_gpu(kernels):
    from imfvideo_b200.config import preset
    from imfvideo_b200.train import Trainer

    cfg = preset("d256")
    cfg.model.depth, cfg.model.aux_head_depth = 3, 1
    cfg.data.latent_frames, cfg.data.latent_size = 4, (16, 32)
    cfg.optim.warmup_steps = 0
    tr = Trainer(cfg, device=torch.device("cuda", 0), verbose=False)
    x, y = torch.randn(1, 16, 4, 16, 32).pin_memory(), torch.randint(0, 1000, (1,))
    st = [tr.train_step(x, y) for _ in range(3)]
    kernels.check_status()
    assert all(s["loss"] == s["loss"] and not s["skipped"] for s in st)
    assert st[-1]["grad_norm"] > 0


@pytest.mark.parametrize("name", ["d256", "d256_sla2"])
def test_train_step_is_bitwise_repeatable(kernels, name):
    """With ``run.deterministic`` two trainers built from the same seed and fed the same batches
    end with bit-identical losses and parameters: every reduction of the step has a fixed
    order (split-K, column sums, dQ accumulation, gradient norm)."""
    from imfvideo_b200.config import preset
    from imfvideo_b200.train import Trainer

    def run():
        cfg = preset(name)
        cfg.model.depth, cfg.model.aux_head_depth = 3, 1
        cfg.data.latent_frames, cfg.data.latent_size = 4, (32, 32)
        cfg.optim.warmup_steps = 0
        cfg.run.deterministic = True
        tr = Trainer(cfg, device=torch.device("cuda", 0), verbose=False)
        g = torch.Generator().manual_seed(7)
        out = []
        for _ in range(2):
            x = torch.randn(1, 16, 4, 32, 32, generator=g).pin_memory()
            y = torch.randint(0, 1000, (1,), generator=g)
            out.append(tr.train_step(x, y))
        flat = torch.cat([p.detach().float().flatten() for p in tr.net.parameters()])
        return out, flat

    try:
        (s1, p1), (s2, p2) = run(), run()
    finally:
        kernels.set_deterministic(False)
    kernels.check_status()
    assert [s["loss"] for s in s1] == [s["loss"] for s in s2]
    assert [s["grad_norm"] for s in s1] == [s["grad_norm"] for s in s2]
    assert torch.equal(p1, p2)


def test_weight_copies_follow_the_optimizer_kernels(kernels):
    """The optimizer's apply kernels and QK-clip write the parameters through raw pointers;
    the blocks' cached bf16 weight copies (gradient-free passes, and the pass under autograd
    when the weight gradients go straight to their buffers) must be rebuilt after each
    step: after two steps the copies a gradient-free pass gets equal the current weights,
    and the step's own passes used the weights of that step (the copies of step 2 differ
    from those of step 1)."""
    from imfvideo_b200.config import preset
    from imfvideo_b200.train import Trainer

    cfg = preset("d256")
    cfg.model.depth, cfg.model.aux_head_depth = 2, 1
    cfg.data.latent_frames, cfg.data.latent_size = 4, (32, 32)
    cfg.optim.warmup_steps = 0
    tr = Trainer(cfg, device=torch.device("cuda", 0), verbose=False)
    blocks = [m for m in tr.net.modules() if hasattr(m, "fused_params")]
    g = torch.Generator().manual_seed(3)
    seen = []
    for _ in range(2):
        x = torch.randn(1, 16, 4, 32, 32, generator=g).pin_memory()
        y = torch.randint(0, 1000, (1,), generator=g)
        st = tr.train_step(x, y)
        assert not st["skipped"]
        assert all(getattr(b, "_wcache", None) is not None for b in blocks)     # the fused path ran
        seen.append([b._wcache[1][1].clone() for b in blocks])
    kernels.check_status()
    assert all(not torch.equal(a, b) for a, b in zip(*seen))
    with torch.no_grad():
        for b in blocks + [m for m in tr.ema.modules() if hasattr(m, "fused_params")]:
            mats = b.fused_params(True)
            assert torch.equal(mats[-5], b.attn.q_b_proj.weight.to(torch.bfloat16))
            f = b.mlp.w2.weight.shape[1]                       # the copy is padded to 8 columns
            assert torch.equal(mats[-1][:, :f], b.mlp.w2.weight.to(torch.bfloat16))


@pytest.mark.parametrize("bs,wide", [(0, False), (2, False), (2, True)])
def test_fused_block_matches_generic_composition(kernels, bs, wide):
    """Same bf16 kernels for GEMM/attention; fused block node vs op-by-op path:
    outputs, tangent and every parameter gradient."""
    from imfvideo_b200.ops import cuda as cu
    from imfvideo_b200.ops.dual import Dual

    net = _net(torch.bfloat16, bs=bs, wide=wide)
    if wide:
        blk = net.shared_blocks[0]
        assert blk.attn.qk_head_dim == 128 and blk.fused_ok(torch.zeros(1, device="cuda"),
                                                            torch.bfloat16)
    B = 2
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(B, 16, 4, 16, 32, device="cuda", generator=g)
    dx = torch.randn(B, 16, 4, 16, 32, device="cuda", generator=g)
    h = torch.rand(B, device="cuda", generator=g)
    w = 1 + torch.rand(B, device="cuda", generator=g)
    lo, hi = torch.zeros(B, device="cuda"), torch.ones(B, device="cuda")
    y = torch.randint(0, 1000, (B,), device="cuda")

    def run():
        net.zero_grad()
        out = net.forward_dual(Dual(x, dx), Dual(h, torch.ones_like(h)), w, lo, hi, y)
        (out["u"].p.square().sum() + out["v"].p.square().sum()).backward()
        return out, {n: p.grad.clone() for n, p in net.named_parameters() if p.grad is not None}

    out_f, g_f = run()
    kernels.check_status()
    cu.disable("block")
    try:
        out_g, g_g = run()
    finally:
        cu.enable("block")
    rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()
    assert rel(out_f["u"].p, out_g["u"].p) < 2e-2 and rel(out_f["v"].p, out_g["v"].p) < 2e-2
    assert rel(out_f["u"].t, out_g["u"].t) < 3e-2
    bad = [(n, rel(g_f[n], g_g[n])) for n in g_g if n in g_f and g_g[n].norm() > 0
           and rel(g_f[n], g_g[n]) > 6e-2]
    assert not bad, bad
    assert set(g_f) >= set(g_g)


def test_weight_gradients_written_straight_into_existing_grad_buffers(kernels):
    """With fp32 ``.grad`` buffers already attached (the optimizer engine's arena views), the
    block node accumulates dY^T X into them itself and hands autograd nothing for the
    matrices; the result equals the autograd route and accumulates over two backward passes."""
    from imfvideo_b200.ops.dual import Dual

    net = _net(torch.bfloat16, bs=2)
    B = 1
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(B, 16, 4, 16, 32, device="cuda", generator=g)
    dx = torch.randn(B, 16, 4, 16, 32, device="cuda", generator=g)
    h = torch.rand(B, device="cuda", generator=g)
    w = 1 + torch.rand(B, device="cuda", generator=g)
    lo, hi = torch.zeros(B, device="cuda"), torch.ones(B, device="cuda")
    y = torch.randint(0, 1000, (B,), device="cuda")

    def backward_once():
        out = net.forward_dual(Dual(x, dx), Dual(h, torch.ones_like(h)), w, lo, hi, y)
        (out["u"].p.square().sum() + out["v"].p.square().sum()).backward()

    net.zero_grad()                       # grads None: gradients travel through autograd
    backward_once()
    via_autograd = {n: p.grad.clone() for n, p in net.named_parameters()}
    for p in net.parameters():            # attached buffers: direct accumulation
        p.grad = torch.zeros_like(p)
    assert net.shared_blocks[0].fused_sinks().direct()
    n0 = kernels.LAUNCHES.count
    backward_once()
    backward_once()
    assert kernels.LAUNCHES.count > n0
    kernels.check_status()
    rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()
    bad = [(n, rel(p.grad, 2 * via_autograd[n])) for n, p in net.named_parameters()
           if via_autograd[n].norm() > 0 and rel(p.grad, 2 * via_autograd[n]) > 1e-2]
    assert not bad, bad


def test_qk_clip_kernel_matches_formula():
    """One-launch QK-Clip over all attention modules against the per-module formula."""
    import math

    from imfvideo_b200 import train as T
    from imfvideo_b200.models import imf_dit_video as M

    torch.manual_seed(0)
    net = M.IMFDiTVideo(input_size=8, num_frames=4, patch_size=(1, 2, 2), in_channels=4,
                        hidden_size=128, depth=3, aux_head_depth=1, num_heads=2,
                        num_classes=10).cuda()
    mods = [m for m in net.modules() if isinstance(m, M.MLAAttention)]
    before = [m.q_b_proj.weight.detach().clone() for m in mods]
    tau = 5.0
    for i, m in enumerate(mods):
        class _Impl:
            pass
        impl = _Impl()
        impl.logit_max_log2 = torch.tensor([3.0 + 4.0 * i, 12.0 - i], device="cuda")
        m.attn_impl = impl
    n, mx = T.qk_clip(net, tau, world=1)
    exp_n, exp_mx = 0, 0.0
    for m, w0 in zip(mods, before):
        s_nat = m.attn_impl.logit_max_log2 * math.log(2.0)
        gamma = (tau / s_nat).clamp(max=1.0)
        exp_n += int((gamma < 1).sum())
        exp_mx = max(exp_mx, float(s_nat.max()))
        ref = w0.view(m.num_heads, m.qk_head_dim, -1).clone()
        ref[:, m.qk_nope_head_dim:, :] *= gamma.view(-1, 1, 1)
        assert torch.allclose(m.q_b_proj.weight.view_as(ref), ref, rtol=1e-6, atol=0)
    assert n == exp_n and abs(mx - exp_mx) < 1e-4


def test_launches_per_block_are_bounded(kernels):
    """Launch accounting (the reference checks its fused launch counts the same way): one
    transformer block of the dual pass is at most 14 launches of this library, a primal-only
    block at most 13, whatever the sequence length; the sequence build (scalar embeddings,
    patch rows) and the output head (re-mix + norm, projection, patch scatter) add a fixed
    number."""
    from imfvideo_b200.ops.dual import Dual

    net = _net(torch.bfloat16)
    B = 1
    x = torch.randn(B, 16, 4, 16, 32, device="cuda")
    h = torch.rand(B, device="cuda")
    w, lo, hi = torch.ones(B, device="cuda") * 1.5, torch.zeros(B, device="cuda"), torch.ones(B, device="cuda")
    y = torch.randint(0, 1000, (B,), device="cuda")
    n_blocks_u = len(net.shared_blocks) + len(net.u_heads)
    with torch.no_grad():
        net.forward_dual(Dual(x, torch.randn_like(x)), Dual(h, torch.ones_like(h)), w, lo, hi, y,
                         branches=("u",), tangent_branches=("u",))       # warm-up
        n0 = kernels.LAUNCHES.count
        net.forward_dual(Dual(x, torch.randn_like(x)), Dual(h, torch.ones_like(h)), w, lo, hi, y,
                         branches=("u",), tangent_branches=("u",))
        dual = kernels.LAUNCHES.count - n0
        n0 = kernels.LAUNCHES.count
        net.forward_dual(Dual(x), Dual(h), w, lo, hi, y, branches=("u",))
        primal = kernels.LAUNCHES.count - n0
    kernels.check_status()
    assert 0 < dual <= 14 * n_blocks_u + 20, dual
    assert 0 < primal <= 13 * n_blocks_u + 20, primal


def test_attention_kernels_stay_finite_on_large_logits(kernels):
    """Stress input (scores far outside the usual range, as in the reference's x10-x100
    battery): forward, tangent and backward stay finite and match the fp32 formulas."""
    from imfvideo_b200.ops import reference as ref

    torch.manual_seed(1)
    B, L, H = 1, 700, 2
    q, k, v, dq, dk, dv, go = (torch.randn(B, L, H, 64, device="cuda") for _ in range(7))
    q, k = q * 12.0, k * 12.0                 # logits of the order of +-150 after the 1/8 scale
    bf = lambda t: t.bfloat16()
    o, do, lse = kernels.attn_fwd(bf(q), bf(k), bf(v), bf(dq), bf(dk), bf(dv))
    gq, gk, gv = kernels.attn_bwd(bf(q), bf(k), bf(v), o, lse, bf(go))
    kernels.check_status()
    for t in (o, do, lse, gq, gk, gv):
        assert torch.isfinite(t.float()).all()
    f = lambda t: bf(t).float()
    o_ref, do_ref = ref.attention_jvp(f(q), f(k), f(v), f(dq), f(dk), f(dv))
    assert (o.float() - o_ref).abs().max() < 3e-2
    assert ((do.float() - do_ref).norm() / do_ref.norm()) < 2e-2


def test_sla2_trainer_steps_finite(kernels):
    """Cube SLA2 INT8-QAT model end to end on the kernels: finite loss and gradients over a
    few seeds (reference tests/test_sla2_e2e.py)."""
    from imfvideo_b200.config import preset
    from imfvideo_b200.train import Trainer

    cfg = preset("d256_sla2")
    cfg.model.depth, cfg.model.aux_head_depth = 3, 1
    cfg.data.latent_frames, cfg.data.latent_size = 4, (16, 32)
    cfg.optim.warmup_steps = 0
    tr = Trainer(cfg, device=torch.device("cuda", 0), verbose=False)
    for seed in range(3):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(1, 16, 4, 16, 32, generator=g).pin_memory()
        y = torch.randint(0, 1000, (1,), generator=g)
        st = tr.train_step(x, y)
        assert st["loss"] == st["loss"] and not st["skipped"], st
        assert st["grad_norm"] == st["grad_norm"] and st["grad_norm"] > 0
    kernels.check_status()


def test_layout_kernels_match_formulas(kernels):
    """Patch gather / scatter (both feature orders, bf16 and fp32), row permutation and the
    sinusoid kernel against the reshape / index / torch formulas, forward and backward."""
    from imfvideo_b200.ops import patch as PK
    from imfvideo_b200.models.imf_dit_video import sinusoid

    assert PK.AVAILABLE
    torch.manual_seed(3)
    B, C, T, H, W, patch = 2, 16, 6, 8, 12, (1, 2, 2)
    for dt in (torch.float32, torch.bfloat16):
        for c_last in (False, True):
            x = torch.randn(B, C, T, H, W, device="cuda").to(dt).requires_grad_(True)
            rows = PK.patch_rows(x, patch, c_last)
            ref = PK.gather_formula(x.detach(), patch, c_last)
            assert rows.dtype == dt and torch.equal(rows, ref)
            g = torch.randn_like(rows)
            rows.backward(g)
            assert torch.equal(x.grad, PK.scatter_formula(g.float(), x.shape, patch, c_last).to(dt))
            r2 = rows.detach().clone().requires_grad_(True)
            vid = PK.unpatch_rows(r2, x.shape, patch, c_last)
            assert vid.dtype == torch.float32 and torch.equal(vid, x.detach().float())
            gv = torch.randn_like(vid)
            vid.backward(gv)
            assert torch.equal(r2.grad, PK.gather_formula(gv, patch, c_last).to(dt))
    L, D = 1000, 256
    z = torch.randn(B, L, D, device="cuda", requires_grad=True)
    perm = torch.randperm(L, device="cuda")
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(L, device="cuda")
    y = PK.permute_rows(z, perm, inv)
    assert torch.equal(y, z.detach()[:, perm])
    gy = torch.randn_like(y)
    y.backward(gy)
    assert torch.equal(z.grad, gy[:, inv])
    zb = torch.randn(B, L, D, device="cuda").bfloat16()
    assert torch.equal(PK.permute_rows(zb, inv, perm), zb[:, inv])
    t = torch.rand(5, device="cuda") * 3
    emb, demb = PK.sinusoid(t, 256)
    half = 128
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device="cuda", dtype=torch.float32) / half)
    arg = t[:, None] * freqs[None]
    assert torch.allclose(emb, torch.cat([arg.cos(), arg.sin()], -1), atol=1e-5)
    assert torch.allclose(demb, torch.cat([-arg.sin() * freqs, arg.cos() * freqs], -1), atol=1e-5)
    e2, d2 = sinusoid(t, 256)
    assert torch.equal(e2, emb) and torch.equal(d2, demb)


def test_newton_schulz_cuda_graph_matches_eager(kernels):
    """The optimizer's Newton-Schulz phase replayed as a CUDA graph (captured on the second
    step) writes exactly the updates of the eager launches, and training steps through it."""
    from imfvideo_b200.config import preset
    from imfvideo_b200.train import Trainer

    cfg = preset("d256")
    cfg.model.depth, cfg.model.aux_head_depth = 2, 1
    cfg.data.latent_frames, cfg.data.latent_size = 4, (16, 32)
    cfg.optim.warmup_steps = 0
    cfg.optim.ns_cuda_graph = True
    tr = Trainer(cfg, device=torch.device("cuda", 0), verbose=False)
    eng = tr.grad_sync
    for seed in range(4):
        g = torch.Generator().manual_seed(100 + seed)
        x = torch.randn(1, 16, 4, 16, 32, generator=g)
        y = torch.randint(0, 1000, (1,), generator=g)
        st = tr.train_step(x, y)
        assert st["loss"] == st["loss"] and not st["skipped"], st
        assert (eng._ns_graph is not None) == (seed >= 1)
    assert eng._ns_graph_launches > 0
    g0 = next(g for g, _ in eng.muon)
    n0 = kernels.LAUNCHES.count
    eng.U.zero_()
    eng._ns_graph.replay()
    u_graph = eng.U.clone()
    eng.U.zero_()
    eng._newton_schulz_eager(tr.optimizer, g0)
    assert kernels.LAUNCHES.count - n0 == eng._ns_graph_launches
    kernels.check_status()
    assert u_graph.float().abs().sum() > 0
    assert torch.equal(u_graph, eng.U)
