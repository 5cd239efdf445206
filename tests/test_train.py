"""CPU: trainer runtime -- schedule, lr groups, QK-clip, EMA, non-finite skip,
atomic checkpoint / resume, config overrides, dataset."""
import math
import os

import pytest
import torch

from imfvideo_b200 import config as C
from imfvideo_b200.config import preset
from imfvideo_b200.data import LatentDataset
from imfvideo_b200.train import Trainer, apply_lr_width_groups, build_model, lr_at, qk_clip
from imfvideo_b200.utils import checkpoint as CK
from imfvideo_b200.utils.schedule import lr_at as lr_fn


def _cfg(tmp_path=None):
    cfg = preset("tiny")
    cfg.optim.muon_coeff_mode = "jordan"
    cfg.run.ema_decay = 0.9
    if tmp_path is not None:
        cfg.run.out_dir = str(tmp_path)
    return cfg


def test_lr_schedule_shapes():
    o = preset("tiny").optim
    o.lr, o.warmup_steps, o.total_steps, o.decay_fraction, o.min_lr_ratio = 1.0, 10, 100, 0.2, 0.1
    assert lr_fn(0, o) == 0 and lr_fn(5, o) == 0.5 and lr_fn(10, o) == 1.0 and lr_fn(79, o) == 1.0
    assert abs(lr_fn(85, o) - (0.1 + 0.9 * (1 - math.sqrt(0.25)))) < 1e-9
    assert abs(lr_fn(100, o) - 0.1) < 1e-9 and abs(lr_fn(1000, o) - 0.1) < 1e-9
    o.decay_shape = "cosine"
    assert abs(lr_fn(90, o) - 0.55) < 1e-9
    o.lr_schedule = "cosine"
    assert abs(lr_fn(55, o) - 0.55) < 1e-9


def test_config_overrides_and_dict_roundtrip():
    cfg = preset("tiny")
    C.apply_overrides(cfg, {"model.hidden_size": "128", "optim": {"lr": 1e-3},
                            "data.latent_size": "(8, 8)", "loss.autocast_bf16": "true"})
    assert cfg.model.hidden_size == 128 and cfg.optim.lr == 1e-3
    assert cfg.data.latent_size == (8, 8) and cfg.loss.autocast_bf16 is True
    with pytest.raises(KeyError):
        C.apply_overrides(cfg, {"model.hiden_size": 1})
    d = C.config_as_dict(cfg)
    cfg2 = C.load_config_dict(preset("tiny"), d)
    assert C.config_as_dict(cfg2) == d
    cfg3 = C.parse_cli(["optim.lr=5e-4", "--model.depth=3"], preset("tiny"))
    assert cfg3.optim.lr == 5e-4 and cfg3.model.depth == 3


def test_lr_width_groups():
    cfg = _cfg()
    cfg.model.hidden_size, cfg.model.attn_res_block_size = 128, 1
    cfg.model.kv_lora_rank = 32
    tr = Trainer(cfg, verbose=False)
    mults = sorted({(g["use_muon"], round(g["lr_width_mult"], 4)) for g in tr.optimizer.param_groups})
    assert mults == [(False, 1.0), (False, 2.0), (True, round(2 ** 0.5, 4)), (True, 2.0)]
    names = {id(p): n for n, p in tr.net.named_parameters()}
    for g in tr.optimizer.param_groups:
        for p in g["params"]:
            n = names[id(p)]
            if g["use_muon"]:
                assert ("_res_proj" in n) == (g["lr_width_mult"] == 2.0)
            elif g["lr_width_mult"] == 2.0:
                assert "final_layer.linear" in n


def test_train_steps_ema_and_resume(tmp_path):
    cfg = _cfg(tmp_path)
    cfg.optim.warmup_steps = 0
    tr = Trainer(cfg, verbose=False)
    x, y = torch.randn(2, 16, 4, 16, 16), torch.randint(0, 1000, (2,))
    w0 = [p.detach().clone() for p in tr.net.parameters()]
    for _ in range(3):
        st = tr.train_step(x, y)
    assert math.isfinite(st["loss"]) and not st["skipped"] and tr.step == 3
    moved = sum(int(not torch.equal(a, b)) for a, b in zip(w0, tr.net.parameters()))
    assert moved > 0.9 * len(w0)
    assert any(not torch.equal(a, b) for a, b in zip(tr.ema.parameters(), tr.net.parameters()))
    path = tr.save()
    assert os.path.basename(path) == "step_0000003.pt"
    ck = torch.load(path, weights_only=True)            # plain containers only
    assert set(ck) >= {"model", "optimizer", "ema", "step", "config"}
    tr2 = Trainer(_cfg(tmp_path), verbose=False)
    tr2.load(path)
    assert tr2.step == 3
    for a, b in zip(tr.net.parameters(), tr2.net.parameters()):
        assert torch.equal(a, b)
    torch.manual_seed(5)
    s1 = tr.train_step(x, y)
    torch.manual_seed(5)
    s2 = tr2.train_step(x, y)
    assert abs(s1["loss"] - s2["loss"]) < 1e-6 and abs(s1["grad_norm"] - s2["grad_norm"]) < 1e-5


def test_resume_keeps_schedule_and_width_multipliers(tmp_path):
    """After a resume the optimizer's param-group dicts are new objects: the update must
    use the scheduled lr x width multiplier written into THEM, so one post-resume step is
    bit-equal (weights, EMA, moments) to the uninterrupted run."""
    def mk():
        cfg = _cfg(tmp_path)
        cfg.optim.warmup_steps = 100
        cfg.model.hidden_size, cfg.model.kv_lora_rank = 128, 32     # width multipliers != 1
        return cfg
    tr = Trainer(mk(), verbose=False)
    x, y = torch.randn(2, 16, 4, 16, 16), torch.randint(0, 1000, (2,))
    for _ in range(3):
        tr.train_step(x, y)
    path = tr.save(sampler_state={"epoch": 2, "batch": 5})
    tr2 = Trainer(mk(), verbose=False)
    tr2.load(path)
    assert tr2.resume_sampler == {"epoch": 2, "batch": 5}
    ck = torch.load(path, weights_only=True)
    assert ck["extra"]["muon_owner"] == tr.grad_sync.owner_table()
    torch.manual_seed(11)
    tr.train_step(x, y)
    torch.manual_seed(11)
    tr2.train_step(x, y)
    lrs = sorted({g["lr"] for g in tr2.optimizer.param_groups})
    assert len(lrs) > 1 and max(lrs) < 2e-3 * 4 / 100 * 2.01          # warm-up lr, not the base lr
    for (n, a), b in zip(tr.net.named_parameters(), tr2.net.parameters()):
        assert torch.equal(a, b), n
    for a, b in zip(tr.ema.parameters(), tr2.ema.parameters()):
        assert torch.equal(a, b)
    for g in tr2.optimizer.param_groups:                               # engine sees the live groups
        assert any(g is eg for eg, _ in tr2.grad_sync.muon + tr2.grad_sync.adam)


def test_infinite_loader_position_roundtrip():
    from imfvideo_b200.data import InfiniteLoader

    data = list(range(7))
    it = InfiniteLoader(data)
    seen = [next(it) for _ in range(10)]               # 7 of epoch 0, 3 of epoch 1
    st = it.state()
    assert st == {"epoch": 1, "batch": 3}
    it2 = InfiniteLoader(data)
    it2.restore(st)
    assert [next(it2) for _ in range(5)] == [next(it) for _ in range(5)]
    assert InfiniteLoader(data).state() == {"epoch": 0, "batch": 0}


def test_checkpoint_is_atomic_and_corruption_is_reported(tmp_path):
    cfg = _cfg(tmp_path)
    tr = Trainer(cfg, verbose=False)
    path = tr.save()
    assert not [f for f in os.listdir(tmp_path) if ".tmp." in f]
    assert CK.latest_checkpoint(str(tmp_path)) == path
    bad = os.path.join(tmp_path, "step_0000009.pt")
    with open(path, "rb") as fh:
        blob = fh.read()
    with open(bad, "wb") as fh:
        fh.write(blob[: len(blob) // 2])              # a kill in mid-write
    with pytest.raises(RuntimeError, match="unreadable"):
        tr.load(bad)
    tr.load(path)


def test_nonfinite_gradient_skips_step(tmp_path):
    cfg = _cfg(tmp_path)
    cfg.optim.warmup_steps = 0
    tr = Trainer(cfg, verbose=False)
    x, y = torch.randn(2, 16, 4, 16, 16), torch.randint(0, 1000, (2,))
    tr.micro_step(x, y)
    next(tr.net.parameters()).grad.view(-1)[0] = float("nan")     # host-side fault injection
    w0 = [p.detach().clone() for p in tr.net.parameters()]
    st = tr.optimizer_step()
    assert st["skipped"]
    for a, b in zip(w0, tr.net.parameters()):
        assert torch.equal(a, b)


def test_qk_clip_scales_rope_rows_only():
    cfg = _cfg()
    net, _, _ = build_model(cfg)
    blk = net.shared_blocks[0].attn

    class Impl:
        logit_max_log2 = torch.tensor([100.0 / math.log(2.0), 10.0])   # head 0 hot: 100 nats

        def __call__(self, q, k, v):
            raise AssertionError

    blk.attn_impl = Impl()
    w0 = blk.q_b_proj.weight.detach().clone().view(2, blk.qk_head_dim, -1)
    hot, smax = qk_clip(net, tau=40.0)
    w1 = blk.q_b_proj.weight.detach().view(2, blk.qk_head_dim, -1)
    dn = blk.qk_nope_head_dim
    assert hot == 1 and abs(smax - 100.0) < 1e-3
    assert torch.allclose(w1[0, dn:], w0[0, dn:] * 0.4) and torch.equal(w1[0, :dn], w0[0, :dn])
    assert torch.equal(w1[1], w0[1])


def _hot_impl():
    class Impl:
        logit_max_log2 = torch.tensor([100.0 / math.log(2.0), 10.0])   # head 0 hot: 100 nats

        def __call__(self, q, k, v):
            raise AssertionError
    return Impl()


def test_qk_clip_respects_skip_flag_and_nonfinite_stats():
    cfg = _cfg()
    net, _, _ = build_model(cfg)
    blk = net.shared_blocks[0].attn
    blk.attn_impl = _hot_impl()
    w0 = blk.q_b_proj.weight.detach().clone()
    hot, _ = qk_clip(net, tau=40.0, skip=torch.tensor([0.0, 1.0]))      # skipped step
    assert hot == 0 and torch.equal(blk.q_b_proj.weight, w0)
    blk.attn_impl.logit_max_log2 = torch.tensor([float("inf"), float("nan")])
    hot, smax = qk_clip(net, tau=40.0, skip=torch.tensor([1.0, 0.0]))
    assert hot == 0 and torch.equal(blk.q_b_proj.weight, w0) and math.isfinite(smax)


def test_qk_clip_ema_matches_reference_order():
    """Reference order is step -> clip -> EMA.  The engine folds the EMA into the update
    kernels (before the clip), so the clip must correct the EMA rows it rescales."""
    import copy
    cfg = _cfg()
    net, _, _ = build_model(cfg)
    ema = copy.deepcopy(net)
    for p in ema.parameters():
        p.data.add_(0.01)
    e0 = copy.deepcopy(ema)
    ema_w = 0.1
    blk = net.shared_blocks[0].attn
    blk.attn_impl = _hot_impl()
    # engine order: EMA absorbs the un-clipped weights first ...
    for pe, p in zip(ema.parameters(), net.parameters()):
        pe.data.lerp_(p.data, ema_w)
    # ... then the clip rescales weights and corrects the EMA
    qk_clip(net, tau=40.0, ema=ema, ema_w=ema_w)
    # reference order on the same start: clip was applied to `net` above, then lerp
    for pe, p in zip(e0.parameters(), net.parameters()):
        pe.data.lerp_(p.data, ema_w)
    for (n, a), b in zip(ema.named_parameters(), e0.parameters()):
        assert torch.allclose(a, b, atol=1e-7), n


def test_skipped_step_keeps_adamw_count_without_train_step(tmp_path):
    """``optimizer_step`` alone (no ``train_step``) after a non-finite gradient: the count
    the update uses lives on the device and does not move on a skipped step."""
    cfg = _cfg(tmp_path)
    cfg.optim.warmup_steps = 0
    tr = Trainer(cfg, verbose=False)
    x, y = torch.randn(2, 16, 4, 16, 16), torch.randint(0, 1000, (2,))
    tr.micro_step(x, y)
    tr.optimizer_step()
    tr.micro_step(x, y)
    next(tr.net.parameters()).grad.view(-1)[0] = float("inf")
    tr.optimizer_step()
    assert float(tr.grad_sync.tcount) == 1.0
    tr.grad_sync.sync_step_count()
    p = tr.grad_sync.adam[0][1]
    assert tr.optimizer.state[p]["step"] == 1


def test_synthetic_dataset():
    cfg = preset("tiny")
    ds = LatentDataset(cfg.data)
    a, la = ds[3]
    b, lb = ds[3]
    assert a.shape == (16, 4, 16, 16) and torch.equal(a, b) and la == lb == 3
    assert not torch.equal(a, ds[4][0])


def test_cli_preset_and_overrides():
    from imfvideo_b200 import config as C

    cfg = C.parse_cli(["--preset", "d256", "optim.total_steps=7", "model.depth=3"], C.Config())
    assert cfg.model.hidden_size == 256 and cfg.model.num_heads == 4
    assert cfg.data.latent_size == (56, 104) and cfg.data.latent_frames == 20
    assert cfg.optim.total_steps == 7 and cfg.model.depth == 3
    assert cfg.model.grad_checkpoint is False


def test_optimizer_step_moves_version_counters_and_refreshes_weight_caches(tmp_path):
    """The flat engine writes parameters through its arenas (a parameter's ``.data`` is a
    view with a version counter of its own), so the step itself must move the counters:
    the blocks key their cached bf16 weight copies for gradient-free passes on them, and a
    stale copy would feed the tangent / guidance passes the weights of an earlier step."""
    cfg = _cfg(tmp_path)
    cfg.optim.warmup_steps = 0
    tr = Trainer(cfg, verbose=False)
    x, y = torch.randn(2, 16, 4, 16, 16), torch.randint(0, 1000, (2,))
    blk = next(m for m in tr.net.modules() if hasattr(m, "fused_params"))
    with torch.no_grad():
        first = blk.fused_params(False)
        again = blk.fused_params(False)
    assert all(a is b for a, b in zip(first[-6:], again[-6:]))          # cached while unchanged
    v0 = [p._version for p in tr.net.parameters()]
    e0 = [p._version for p in tr.ema.parameters()]
    st = tr.train_step(x, y)
    assert not st["skipped"]
    assert all(p._version > v for p, v in zip(tr.net.parameters(), v0))
    assert all(p._version > v for p, v in zip(tr.ema.parameters(), e0))
    with torch.no_grad():
        after = blk.fused_params(False)
    w_qb = blk.attn.q_b_proj.weight
    assert torch.equal(after[-5], w_qb.to(torch.bfloat16))
    assert not torch.equal(first[-5].float(), after[-5].float())


def test_mark_written_moves_counters_without_touching_data():
    from imfvideo_b200.utils import mark_written

    a, b = torch.arange(4.0), torch.nn.Parameter(torch.ones(3))
    va, vb = a._version, b._version
    mark_written([a, None, b])
    assert a._version > va and b._version > vb
    assert torch.equal(a, torch.arange(4.0)) and torch.equal(b.detach(), torch.ones(3))
    mark_written([])


def test_weight_copies_under_autograd_follow_the_gradient_buffers():
    """With fp32 gradient buffers on every parameter the fused block writes its weight
    gradients straight into them, so the bf16 weight copies carry no autograd history and are
    shared with the gradient-free passes; without the buffers autograd has to carry the
    gradients back through the copies, which are then rebuilt with history on every call."""
    cfg = _cfg()
    cfg.model.attn_res_block_size = 2           # blocks with the attention-residual re-mix
    net = build_model(cfg)[0]
    blk = next(m for m in net.modules() if hasattr(m, "fused_params") and hasattr(m, "attn_res_norm"))
    with torch.no_grad():
        cached = blk.fused_params(False)[-6:]
    # no gradient buffers yet: the copies must be differentiable
    mats = blk.fused_params(False)[-6:]
    assert all(m.requires_grad for m in mats) and not blk.fused_sinks().mats_cached
    for p in blk.parameters():
        p.grad = torch.zeros_like(p)
    mats = blk.fused_params(False)[-6:]
    assert blk.fused_sinks().direct() and blk.fused_sinks().mats_cached
    assert all((not m.requires_grad) and m is c for m, c in zip(mats, cached))
    # the small products of two parameters keep their history under autograd
    w1, w2 = blk.fused_params(True)[:2]
    assert w1.requires_grad and w2.requires_grad
    with torch.no_grad():
        a1, _ = blk.fused_params(True)[:2]
        b1, _ = blk.fused_params(True)[:2]
    assert a1 is b1 and not a1.requires_grad and torch.equal(a1, w1.detach())
