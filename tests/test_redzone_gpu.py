"""GPU: out-of-bounds writes.  compute-sanitizer is not available where these tests run, so
each kernel here writes into a view that sits between two guard regions filled with a
sentinel; after the launch the guards must be intact.  Shapes are ragged on purpose (rows
and columns that do not fill the last tile)."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
SENTINEL = {torch.bfloat16: -7.75, torch.float32: -12345.5}


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from imfvideo_b200.ops import cuda as cu

    assert cu.available()
    from imfvideo_b200.ops import kernels

    return kernels


class Guarded:
    """A tensor of ``shape`` carved out of a larger buffer, ``pad`` sentinel elements on
    each side (pad keeps the view 256-byte aligned)."""

    def __init__(self, shape, dtype, pad=4096):
        n = math.prod(shape)
        self.buf = torch.full((n + 2 * pad,), SENTINEL[dtype], dtype=dtype, device="cuda")
        self.t = self.buf[pad:pad + n].view(*shape)
        self.pad, self.n = pad, n

    def intact(self) -> bool:
        s = SENTINEL[self.buf.dtype]
        return bool((self.buf[:self.pad] == s).all() and (self.buf[self.pad + self.n:] == s).all())


@pytest.mark.parametrize("M,N,Kd", [(300, 200, 136), (77, 72, 64), (1000, 528, 256)])
def test_gemm_outputs_stay_inside(K, M, N, Kd):
    torch.manual_seed(0)
    A = torch.randn(M, Kd, device="cuda").bfloat16()
    B = torch.randn(N, Kd, device="cuda").bfloat16()
    for dt in (torch.bfloat16, torch.float32):
        g = Guarded((M, N), dt)
        K.gemm(A, B, out=g.t)
        torch.cuda.synchronize()
        assert g.intact() and (g.t != SENTINEL[dt]).any()
    g = Guarded((N, Kd), torch.float32)
    dy = torch.randn(M, N, device="cuda").bfloat16() if N % 8 == 0 else None
    if dy is not None:
        K.gemm_wgrad(dy, A, out=g.t)
        torch.cuda.synchronize()
        assert g.intact()
    K.check_status()


@pytest.mark.parametrize("hd,L,H", [(64, 333, 3), (128, 333, 3), (64, 2100, 40)])
def test_attention_outputs_stay_inside(K, hd, L, H):
    torch.manual_seed(1)
    B = 1
    q, k, v, go = (torch.randn(B, L, H, hd, device="cuda").bfloat16() for _ in range(4))
    o, lse = Guarded((B, L, H, hd), torch.bfloat16), Guarded((B, H, L), torch.float32)
    nscr = int(K._lib.imf_attn_fwd_scratch_bytes_hd(B, L, H, 0, hd))
    scr = Guarded((max(nscr, 16),), torch.bfloat16) if nscr else None
    strides = []
    for t in (q, k, v):
        strides += [t.stride(0), t.stride(1), t.stride(2)]
    arr = (ctypes.c_int64 * 18)(*(strides + [0] * 9))
    rc = K._lib.imf_attn_fwd(K._ptr(q), K._ptr(k), K._ptr(v), None, None, None, K._ptr(o.t), None,
                             K._ptr(lse.t), B, L, H, hd, ctypes.cast(arr, ctypes.c_void_p),
                             o.t.stride(0), o.t.stride(1), o.t.stride(2), 1.0 / math.sqrt(hd),
                             K._ptr(scr.t) if scr else None, 2 * nscr if scr else 0,
                             K._ptr(K.status_word(q.device)), K._stream())
    assert rc == 0
    torch.cuda.synchronize()
    assert o.intact() and lse.intact() and (scr is None or scr.intact())
    ref, _, ref_lse = K.attn_fwd(q, k, v)
    assert torch.equal(ref, o.t) and torch.equal(ref_lse, lse.t)
    # backward: dv lands in a band of a wider guarded buffer; the rest of it must not change
    wide = Guarded((B, L, H, hd + 48), torch.bfloat16)
    dq, dk, dv = K.attn_bwd(q, k, v, ref, ref_lse, go, gv_out=wide.t[..., 48:])
    torch.cuda.synchronize()
    assert wide.intact() and (wide.t[..., :48] == SENTINEL[torch.bfloat16]).all()
    assert torch.isfinite(dq.float()).all() and torch.isfinite(dk.float()).all()
    K.check_status()
