"""GPU: each sm_100a kernel against the plain-PyTorch fp32 formulas."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from imfvideo_b200.ops import cuda as cu

    assert cu.available(), "kernel library must load on a GPU box"
    from imfvideo_b200.ops import kernels

    return kernels


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("M,N,Kd", [(128, 128, 64), (304, 200, 136), (1000, 528, 256), (77, 64, 8)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm(K, M, N, Kd, a_mn, b_mn):
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operand needs a 16-byte-multiple row stride")
    torch.manual_seed(0)
    A = torch.randn(M, Kd, device="cuda").bfloat16()
    B = torch.randn(N, Kd, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda")
    out = K.gemm(A.t().contiguous() if a_mn else A, B.t().contiguous() if b_mn else B,
                 a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, bias=bias, bias_rows=M // 2)
    ref = A.float() @ B.float().t()
    ref[: M // 2] += bias
    assert _rel(out, ref) < 1e-5
    out16 = K.gemm(A.t().contiguous() if a_mn else A, B.t().contiguous() if b_mn else B,
                   a_mn=a_mn, b_mn=b_mn)
    assert _rel(out16, A.float() @ B.float().t()) < 4e-3
    K.check_status()


@pytest.mark.parametrize("rows,M,N", [(29140, 528, 256), (1000, 144, 256), (4100, 256, 682),
                                      (333, 64, 72), (20000, 1364, 256)])
def test_gemm_weight_gradient_splitk(K, rows, M, N):
    """dY^T X over many token rows: split-K slices summed in a fixed order; strided operand
    views (a band of a wider dY, the first columns of a wider X); accumulation into an
    existing fp32 buffer; two runs give the same bits."""
    torch.manual_seed(rows)
    dy_full = torch.randn(rows, (M + 23) // 8 * 8, device="cuda").bfloat16()
    x_full = torch.randn(rows, (N + 15) // 8 * 8, device="cuda").bfloat16()   # 16-byte row pitch
    dy, x = dy_full[:, 8:8 + M], x_full[:, :N]
    ref = dy.float().t() @ x.float()
    out = K.gemm_wgrad(dy, x)
    assert out.dtype == torch.float32 and _rel(out, ref) < 1e-5
    base = torch.randn(M, N, device="cuda")
    acc = base.clone()
    K.gemm_wgrad(dy, x, out=acc, accumulate=True)
    assert _rel(acc, base + ref) < 1e-5
    assert torch.equal(K.gemm_wgrad(dy, x), out)
    K.check_status()


@pytest.mark.parametrize("M,N,Kd", [(256, 128, 128), (1000, 528, 256), (300, 200, 136), (4096, 768, 1024)])
def test_gemm_fp8(K, M, N, Kd):
    """e4m3 operands on the kind::f8f6f4 tensor path: exact against the same quantised values
    multiplied in fp32, and within the reference's fp8 envelope (4e-2) of the unquantised product."""
    torch.manual_seed(M)
    A = torch.randn(M, Kd, device="cuda").bfloat16()
    B = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(N, device="cuda")
    a8, sa = K.quantize_fp8(A)
    b8, sb = K.quantize_fp8(B)
    assert a8.shape == (M, (Kd + 15) // 16 * 16) and (a8[:, Kd:] == 0).all()
    deq = lambda t8, s_: t8.view(torch.float8_e4m3fn).float() * s_
    assert _rel(deq(a8, sa)[:, :Kd], A) < 4e-2 and float(sa) > 0
    out = K.gemm_fp8(a8, sa, b8, sb, out_dtype=torch.float32, bias=bias)
    exact = deq(a8, sa) @ deq(b8, sb).t() + bias
    assert _rel(out, exact) < 1e-5
    full = A.float() @ B.float().t() + bias
    assert _rel(out, full) < 4e-2
    y = K.linear_fp8(A, B, bias)
    assert y.dtype == torch.bfloat16 and _rel(y, full) < 4e-2
    K.check_status()


@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("M,N,Kd", [(1000, 1024, 1536), (300, 1400, 2736)])
def test_gemm_wide_tiles(K, M, N, Kd, b_mn):
    """Wide and deep products take the 128 x 256 tile instance (ragged M and N included)."""
    torch.manual_seed(N)
    A = torch.randn(M, Kd, device="cuda").bfloat16()
    B = (torch.randn(N, Kd, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda")
    out = K.gemm(A, B.t().contiguous() if b_mn else B, b_mn=b_mn, bias=bias, bias_rows=M // 2)
    ref = A.float() @ B.float().t()
    ref[: M // 2] += bias
    assert _rel(out, ref) < 4e-3
    K.check_status()


def test_gemm_rejects_bad_stride(K):
    A = torch.randn(64, 12, device="cuda").bfloat16()      # K = 12: stride not 16-byte multiple
    with pytest.raises(ValueError):
        K.gemm(A, A)


@pytest.mark.parametrize("B,L,H", [(1, 256, 1), (1, 300, 2), (2, 1000, 3), (1, 64, 1), (1, 2049, 2)])
def test_attention_forward(K, B, L, H):
    from imfvideo_b200.ops import reference as ref

    g = torch.Generator(device="cuda").manual_seed(L)
    q, k, v = (torch.randn(B, L, H, 64, device="cuda", generator=g).bfloat16() for _ in range(3))
    o, _, lse = K.attn_fwd(q, k, v)
    ro = ref.attention(q.float(), k.float(), v.float())
    assert (o.float() - ro).abs().max() < 2e-2 and _rel(o, ro) < 1e-2
    assert (lse - ref.attention_lse(q.float(), k.float())).abs().max() < 1e-3
    K.check_status()


@pytest.mark.parametrize("B,L,H", [(1, 256, 1), (1, 212, 2), (2, 1000, 3), (1, 2049, 2)])
def test_attention_forward_tangent(K, B, L, H):
    from imfvideo_b200.ops import reference as ref

    g = torch.Generator(device="cuda").manual_seed(L)
    mk = lambda s: (torch.randn(B, L, H, 64, device="cuda", generator=g) * s).bfloat16()
    q, k, v, dq, dk, dv = mk(1), mk(1), mk(1), mk(.5), mk(.5), mk(.5)
    o, do, lse = K.attn_fwd(q, k, v, dq, dk, dv)
    ro, rdo = ref.attention_jvp(*(t.float() for t in (q, k, v, dq, dk, dv)))
    assert (o.float() - ro).abs().max() < 2e-2 and _rel(o, ro) < 1e-2
    assert (do.float() - rdo).abs().max() < 2e-2 and _rel(do, rdo) < 1e-2
    o2, _, _ = K.attn_fwd(q, k, v)
    assert _rel(o2, o) < 5e-3            # primal-only and fused kernels agree
    K.check_status()


@pytest.mark.parametrize("B,L,H", [(1, 256, 1), (1, 300, 3), (2, 1000, 3), (1, 64, 1), (1, 2049, 2),
                                   (2, 2100, 12)])
def test_attention_forward_hd128(K, B, L, H):
    """head_dim 128, head counts that are not powers of two, ragged lengths, and (last case)
    more work items than SMs, so items are split between CTAs and merged."""
    from imfvideo_b200.ops import reference as ref

    g = torch.Generator(device="cuda").manual_seed(L)
    q, k, v = (torch.randn(B, L, H, 128, device="cuda", generator=g).bfloat16() for _ in range(3))
    o, _, lse = K.attn_fwd(q, k, v)
    for h in sorted({0, H // 2, H - 1}):
        sl = slice(h, h + 1)
        ro = ref.attention(q[:, :, sl].float(), k[:, :, sl].float(), v[:, :, sl].float())
        assert (o[:, :, sl].float() - ro).abs().max() < 2e-2 and _rel(o[:, :, sl], ro) < 1e-2
        rl = ref.attention_lse(q[:, :, sl].float(), k[:, :, sl].float())
        assert (lse[:, sl] - rl).abs().max() < 1e-3
    K.check_status()


@pytest.mark.parametrize("B,L,H", [(1, 128, 1), (1, 212, 3), (2, 1000, 3), (1, 2049, 2), (1, 2100, 12)])
def test_attention_forward_tangent_hd128(K, B, L, H):
    from imfvideo_b200.ops import reference as ref

    g = torch.Generator(device="cuda").manual_seed(L)
    mk = lambda s: (torch.randn(B, L, H, 128, device="cuda", generator=g) * s).bfloat16()
    q, k, v, dq, dk, dv = mk(1), mk(1), mk(1), mk(.5), mk(.5), mk(.5)
    o, do, lse = K.attn_fwd(q, k, v, dq, dk, dv)
    for h in sorted({0, H // 2, H - 1}):
        sl = slice(h, h + 1)
        ro, rdo = ref.attention_jvp(*(t[:, :, sl].float() for t in (q, k, v, dq, dk, dv)))
        assert (o[:, :, sl].float() - ro).abs().max() < 2e-2 and _rel(o[:, :, sl], ro) < 1e-2
        assert (do[:, :, sl].float() - rdo).abs().max() < 3e-2 and _rel(do[:, :, sl], rdo) < 1e-2
    o2, _, lse2 = K.attn_fwd(q, k, v)
    assert _rel(o2, o) < 5e-3            # primal-only and fused kernels agree
    assert (lse - lse2).abs().max() < 1e-3
    o3, do3, _ = K.attn_fwd(q, k, v, dq, dk, dv)
    assert torch.equal(o, o3) and torch.equal(do, do3)       # run twice: same bits
    K.check_status()


def test_attention_strided_views_and_run_twice(K):
    """v as a slice of a wider kv tensor (as in MLA); two runs are bit-equal."""
    torch.manual_seed(0)
    B, L, H = 1, 515, 4
    kv = torch.randn(B, L, H, 112, device="cuda").bfloat16()
    q = torch.randn(B, L, H, 64, device="cuda").bfloat16()
    k = torch.randn(B, L, H, 64, device="cuda").bfloat16()
    v = kv[..., 48:]
    o1, _, _ = K.attn_fwd(q, k, v)
    o2, _, _ = K.attn_fwd(q, k, v.contiguous())
    o3, _, _ = K.attn_fwd(q, k, v)
    assert torch.equal(o1, o2) and torch.equal(o1, o3)
    K.check_status()


def test_attention_autograd(K):
    from imfvideo_b200.ops import reference as ref
    from imfvideo_b200.ops.dual import Dual

    torch.manual_seed(0)
    B, L, H = 1, 333, 2
    q, k, v = (torch.randn(B, L, H, 64, device="cuda").bfloat16().requires_grad_(True)
               for _ in range(3))
    go = torch.randn(B, L, H, 64, device="cuda").bfloat16()
    out = K.attention_dual(Dual(q), Dual(k), Dual(v)).p
    out.backward(go)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref.attention(qf, kf, vf).backward(go.float())
    for a, b in ((q, qf), (k, kf), (v, vf)):
        assert _rel(a.grad, b.grad) < 2e-2
    K.check_status()


@pytest.mark.parametrize("B,L,H", [(1, 128, 1), (1, 300, 2), (2, 1000, 3), (1, 2049, 2)])
def test_attention_backward(K, B, L, H):
    from imfvideo_b200.ops import reference as ref

    g = torch.Generator(device="cuda").manual_seed(L)
    q, k, v, go = (torch.randn(B, L, H, 64, device="cuda", generator=g).bfloat16() for _ in range(4))
    o, _, lse = K.attn_fwd(q, k, v)
    kvbuf = torch.zeros(B, L, H, 112, dtype=torch.bfloat16, device="cuda")
    dq, dk, dv = K.attn_bwd(q, k, v, o, lse, go, gv_out=kvbuf[..., 48:])
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref.attention(qf, kf, vf).backward(go.float())
    for name, a, b in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        assert _rel(a, b) < 1.5e-2, (name, _rel(a, b))
    assert (kvbuf[..., :48] == 0).all()        # only the value band was written
    dq2, dk2, dv2 = K.attn_bwd(q, k, v, o, lse, go)
    assert torch.equal(dk, dk2) and torch.equal(dv2, dv.contiguous())
    assert _rel(dq2, dq) < 1e-3              # dQ tiles land in arrival order
    K.check_status()
    K.set_deterministic(True)                # fixed order: bit-identical dQ, same values
    try:
        dq3, dk3, dv3 = K.attn_bwd(q, k, v, o, lse, go)
        dq4, _, _ = K.attn_bwd(q, k, v, o, lse, go)
    finally:
        K.set_deterministic(False)
    assert torch.equal(dk3, dk) and torch.equal(dv3, dv.contiguous())
    assert torch.equal(dq3, dq4) and _rel(dq3, dq) < 1e-3
    K.check_status()


@pytest.mark.parametrize("B,L,H", [(1, 128, 1), (1, 300, 3), (2, 1000, 3), (1, 2049, 2), (1, 2100, 12)])
def test_attention_backward_hd128(K, B, L, H):
    """head_dim 128 reverse mode (64-row query steps, transposed dQ tiles); the last case
    splits the query range of each K/V tile over several CTAs."""
    from imfvideo_b200.ops import reference as ref

    g = torch.Generator(device="cuda").manual_seed(L)
    q, k, v, go = (torch.randn(B, L, H, 128, device="cuda", generator=g).bfloat16() for _ in range(4))
    o, _, lse = K.attn_fwd(q, k, v)
    kvbuf = torch.zeros(B, L, H, 224, dtype=torch.bfloat16, device="cuda")
    dq, dk, dv = K.attn_bwd(q, k, v, o, lse, go, gv_out=kvbuf[..., 96:])
    for h in sorted({0, H // 2, H - 1}):
        sl = slice(h, h + 1)
        qf, kf, vf = (t[:, :, sl].float().requires_grad_(True) for t in (q, k, v))
        ref.attention(qf, kf, vf).backward(go[:, :, sl].float())
        for name, a, b in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
            assert _rel(a[:, :, sl], b) < 1.5e-2, (name, h, _rel(a[:, :, sl], b))
    assert (kvbuf[..., :96] == 0).all()        # only the value band was written
    dq2, dk2, dv2 = K.attn_bwd(q, k, v, o, lse, go)
    assert torch.equal(dk, dk2) and torch.equal(dv2, dv.contiguous())
    assert _rel(dq2, dq) < 1e-3
    K.check_status()


@pytest.mark.parametrize("k,n,m", [(3, 128, 256), (2, 256, 128), (2, 256, 682), (2, 682, 256),
                                   (4, 1, 256), (1, 448, 128), (1, 520, 1024)])
def test_newton_schulz_kernel(K, k, n, m):
    from imfvideo_b200.ops import reference as ref

    torch.manual_seed(n + m)
    G = torch.randn(k, n, m, device="cuda")
    coeffs = (3.4445, -4.7750, 2.0315)
    X = K.newton_schulz(G, coeffs, steps=5)
    if n == 1:
        assert X is None            # vectors take the torch path
        return
    assert X.shape == (k, n, m)
    for i in range(k):
        R = ref.newton_schulz(G[i], coeffs, steps=5, dtype=torch.float32)
        assert _rel(X[i], R) < 4e-2, (i, _rel(X[i], R))
    K.check_status()


def test_batched_gemm_with_additive_source(K):
    torch.manual_seed(0)
    a = torch.randn(3, 200, 136, device="cuda").bfloat16()
    b = torch.randn(3, 96, 136, device="cuda").bfloat16()
    cin = torch.randn(3, 200, 96, device="cuda").bfloat16()
    out = K.gemm_batched(a, b, cin=cin, alpha=0.5, beta=2.0)
    ref = 0.5 * torch.einsum("zmk,znk->zmn", a.float(), b.float()) + 2.0 * cin.float()
    assert _rel(out, ref) < 5e-3
    K.check_status()


@pytest.mark.parametrize("n,kdim,mn", [(200, 136, False), (264, 520, True), (1024, 256, False),
                                       (128, 64, False), (392, 1032, True)])
def test_batched_gemm_symmetric_products(K, n, kdim, mn):
    """X X^T / X^T X and b A + c A A with the symmetric mode (upper tiles + mirror image in
    the epilogue) against the full product: the upper triangle is bit-identical, the result
    exactly symmetric, and both agree with fp32."""
    torch.manual_seed(n)
    Z = 3
    x = (torch.randn(Z, kdim, n, device="cuda") if mn else
         torch.randn(Z, n, kdim, device="cuda")).bfloat16() * 0.1
    full = K.gemm_batched(x, x, a_mn=mn, b_mn=mn)
    sym = K.gemm_batched(x, x, a_mn=mn, b_mn=mn, sym=True)
    xf = x.float().transpose(1, 2) if mn else x.float()
    ref = torch.einsum("zik,zjk->zij", xf, xf)
    assert _rel(sym, ref) < 5e-3
    assert torch.equal(sym, sym.transpose(1, 2))
    iu = torch.triu_indices(n, n, device="cuda")
    # tiles on the diagonal are computed whole, tiles above it are the same launches' tiles
    assert torch.equal(sym[:, iu[0], iu[1]], full[:, iu[0], iu[1]])
    b2 = K.gemm_batched(sym, sym, cin=sym, alpha=2.0, beta=-4.75, sym=True)
    ref2 = 2.0 * torch.einsum("zik,zjk->zij", sym.float(), sym.float()) - 4.75 * sym.float()
    assert _rel(b2, ref2) < 5e-3
    assert torch.equal(b2, b2.transpose(1, 2))
    K.check_status()


@pytest.mark.parametrize("hd,B,L,H", [(64, 1, 9000, 4), (128, 1, 6000, 5)])
def test_attention_backward_bitwise_repeatable_over_several_waves(K, hd, B, L, H):
    """More K/V tiles than SMs (several waves of CTAs, split query ranges): the fixed-order dQ
    accumulation gives bit-identical gradients on every run."""
    g = torch.Generator(device="cuda").manual_seed(hd + L)
    q, k, v, go = (torch.randn(B, L, H, hd, device="cuda", generator=g).bfloat16() for _ in range(4))
    o, _, lse = K.attn_fwd(q, k, v)
    loose = K.attn_bwd(q, k, v, o, lse, go)
    K.set_deterministic(True)
    try:
        first = K.attn_bwd(q, k, v, o, lse, go)
        for _ in range(3):
            again = K.attn_bwd(q, k, v, o, lse, go)
            assert all(torch.equal(a, b) for a, b in zip(first, again))
    finally:
        K.set_deterministic(False)
    assert _rel(first[0], loose[0]) < 1e-3
    K.check_status()


@pytest.mark.parametrize("M,N,Kd", [(20480, 528, 256), (29140, 1000, 200), (58280, 264, 64),
                                    (19000, 768, 256)])
def test_gemm_short_k_many_tiles(K, M, N, Kd):
    """Short-K products with many tiles (the projections of a narrow model on a long sequence):
    ragged M, N and K, a strided A, bit-equal repeats."""
    g = torch.Generator(device="cuda").manual_seed(M + N + Kd)
    a_wide = torch.randn(M, Kd + 24, device="cuda", generator=g).bfloat16()
    a = a_wide[:, 8:8 + Kd]                                   # row pitch != K, 16-byte aligned
    b = torch.randn(N, Kd, device="cuda", generator=g).bfloat16()
    out = K.gemm(a, b, alpha=0.5)
    ref = 0.5 * (a.float() @ b.float().t())
    assert _rel(out, ref) < 4e-3
    idx = torch.tensor([0, 127, 128, M // 2, M - 1], device="cuda")
    assert torch.allclose(out[idx].float(), ref[idx], rtol=2e-2, atol=2e-2 * ref.abs().max().item())
    out2 = K.gemm(a, b, alpha=0.5)
    assert torch.equal(out, out2)
    K.check_status()
