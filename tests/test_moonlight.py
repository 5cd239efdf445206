"""CPU: optimizer maths (model of the reference's tests/test_moonlight.py)."""
import copy
import json
import math
import os

import pytest
import torch

from imfvideo_b200.models import IMFDiTVideo
from imfvideo_b200.optim import moonlight as ML


def test_newton_schulz_envelope_and_shape_blindness():
    torch.manual_seed(0)
    for n, m in [(64, 64), (32, 128), (128, 32)]:
        G = torch.randn(n, m)
        X = ML.zeropower_via_newtonschulz5(G, steps=5)
        s = torch.linalg.svdvals(X)
        # a square Gaussian has near-zero singular values that five steps cannot lift
        lo = s.min() if n != m else s.quantile(0.1)
        assert X.shape == (n, m) and 0.6 < lo and s.max() < 1.25
        Xt = ML.zeropower_via_newtonschulz5(G.T.contiguous(), steps=5)
        assert torch.allclose(Xt.T, X, atol=1e-4)
    G3 = torch.randn(3, 48, 96)
    X3 = ML.zeropower_via_newtonschulz5(G3)
    for i in range(3):
        assert torch.allclose(X3[i], ML.zeropower_via_newtonschulz5(G3[i]), atol=1e-5)


def test_coefficient_solver_beats_jordan_and_cache(tmp_path, monkeypatch):
    coeffs, mse = ML.solve_ns_coefficients(32, 96, steps=5, opt_iters=600)
    sigma = ML.sample_normalized_spectrum(32, 96)
    a, b, c = ML.JORDAN_COEFFS
    x = sigma
    for _ in range(5):
        x = a * x + b * x ** 3 + c * x ** 5
    assert mse < float(((x - 1) ** 2).mean())
    path = tmp_path / "c.json"
    monkeypatch.setenv("MOONLIGHT_COEFF_CACHE", str(path))
    ML._COEFF_CACHE.clear()
    c1 = ML.get_ns_coefficients(20, 24, 5, opt_iters=50)
    assert json.load(open(path))["20x24x5"] == list(c1)
    ML._COEFF_CACHE.clear()
    assert ML.get_ns_coefficients(24, 20, 5, opt_iters=50) == tuple(c1)   # disk hit, (n,m)~(m,n)
    assert ML.get_ns_coefficients(3, 3, 5, mode="jordan") == ML.JORDAN_COEFFS


def test_packaged_table_matches_reference_table():
    from conftest import reference_dir

    d = reference_dir()
    ref = os.path.join(d, ".cache", "ns_coeffs.json") if d else ""
    if not os.path.exists(ref):
        pytest.skip("reference cache not available")
    theirs = json.load(open(ref))
    ours = json.load(open(ML._PACKAGED_CACHE))
    common = set(theirs) & set(ours)
    assert common
    for k in common:
        assert all(abs(x - y) < 2e-2 * max(1, abs(y)) for x, y in zip(ours[k], theirs[k])), k


def test_update_rms_is_shape_independent():
    torch.manual_seed(0)
    for n, m in [(64, 64), (32, 256), (256, 48)]:
        p = torch.nn.Parameter(torch.zeros(n, m))
        p.grad = torch.randn(n, m)
        opt = ML.Moonlight([p], [], lr=1.0, weight_decay=0.0, coeff_mode="jordan")
        opt.step()
        rms = p.detach().pow(2).mean().sqrt().item()
        assert 0.14 < rms < 0.26, (n, m, rms)


def _tiny():
    torch.manual_seed(0)
    return IMFDiTVideo(input_size=8, num_frames=2, hidden_size=32, depth=2, num_heads=2,
                       aux_head_depth=1, attn_res_block_size=1)


def test_split_rules():
    net = _tiny()
    names = {id(p): n for n, p in net.named_parameters()}
    muon, adamw = ML.split_params(net)
    mn, an = {names[id(p)] for p in muon}, {names[id(p)] for p in adamw}
    assert "shared_blocks.0.attn.q_a_proj.weight" in mn
    assert "shared_blocks.0.attn.g_proj.weight" in mn
    assert "shared_blocks.0.attn_res_proj.weight" in mn          # Linear(d, 1) score head
    assert "u_out_res_proj.weight" in mn
    for n in ("time_tokens", "x_embedder.proj.weight", "h_embedder.mlp.0.weight",
              "y_embedder.embedding_table.weight", "u_final_layer.linear.weight",
              "shared_blocks.0.attn_scale", "shared_blocks.0.norm1.weight"):
        assert n in an, n
    assert len(mn) + len(an) == len(list(net.parameters()))


def test_adamw_branch_matches_torch():
    torch.manual_seed(0)
    p1 = torch.nn.Parameter(torch.randn(17, 5))
    p2 = torch.nn.Parameter(p1.detach().clone())
    a = ML.Moonlight([], [p1], lr=1e-2, weight_decay=0.1, adamw_betas=(0.9, 0.95))
    b = torch.optim.AdamW([p2], lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-8)
    for _ in range(20):
        g = torch.randn(17, 5)
        p1.grad, p2.grad = g.clone(), g.clone()
        a.step()
        b.step()
    assert (p1 - p2).abs().max() < 1e-5


def test_matches_reference_optimizer(ref_modules):
    R = ref_modules["moonlight"]
    net_a = _tiny()
    net_b = copy.deepcopy(net_a)
    kw = dict(lr=2e-3, weight_decay=0.1, momentum=0.9, coeff_mode="jordan")
    oa = ML.build_moonlight(net_a, **kw)
    ob = R.build_moonlight(net_b, **kw)
    for s in range(3):
        torch.manual_seed(s)
        for pa, pb in zip(net_a.parameters(), net_b.parameters()):
            g = torch.randn_like(pa)
            pa.grad, pb.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    for (n, pa), pb in zip(net_a.named_parameters(), net_b.parameters()):
        assert torch.allclose(pa, pb, atol=2e-6), n
    sa, sb = oa.state_dict(), ob.state_dict()
    assert [g["params"] for g in sa["param_groups"]] == [g["params"] for g in sb["param_groups"]]
    ka = {k: sorted(v) for k, v in sa["state"].items()}
    kb = {k: sorted(v) for k, v in sb["state"].items()}
    assert ka == kb
    ob.load_state_dict(sa)          # interchangeable state dicts


def test_state_dict_roundtrip_and_lr_wiring():
    net = _tiny()
    opt = ML.build_moonlight(net, lr=1e-3, weight_decay=0.1, coeff_mode="jordan")
    for p in net.parameters():
        p.grad = torch.randn_like(p)
    opt.step()
    sd = copy.deepcopy(opt.state_dict())
    opt2 = ML.build_moonlight(copy.deepcopy(net), lr=1e-3, weight_decay=0.1, coeff_mode="jordan")
    opt2.load_state_dict(sd)
    assert opt2.state_dict()["param_groups"][0]["use_muon"] is True
    before = [p.detach().clone() for p in net.parameters()]
    for g in opt.param_groups:
        g["lr"] = 0.0
    opt.step()
    for b, p in zip(before, net.parameters()):
        assert torch.equal(b, p)        # lr drives both branches
