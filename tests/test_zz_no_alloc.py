"""GPU: the allocation-free attention entry point, called through its exported
C symbol exactly as an external caller would.

Who needs it: callers that cannot allocate device memory (no cudaMalloc where
they run, or no allocator of their own) and so cannot provide the scratch
buffer that the regular entry point takes.  The library keeps that scratch in
a built-in device array instead.  This test checks, on two calls in a row
(the array keeps the first call's contents), that the result equals the
regular entry point's and the plain fp32 formula, and that an oversized request
is refused with an error code rather than launched.  The file name sorts last so every other test has
already run if this one fails under ``-x``.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, q, k, v, status):
    B, L, H, hd = q.shape
    o = torch.empty_like(q)
    lse = torch.empty(B, H, L, dtype=torch.float32, device=q.device)
    strides = []
    for t in (q, k, v):
        strides += [t.stride(0), t.stride(1), t.stride(2)]
    arr = (ctypes.c_int64 * 9)(*strides)
    fn = lib.imf_attn_fwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 4 + [ctypes.c_void_p] + \
                  [ctypes.c_int64] * 3 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, L, H, hd,
            ctypes.cast(arr, ctypes.c_void_p), o.stride(0), o.stride(1), o.stride(2),
            1.0 / math.sqrt(hd), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, o, lse


def test_noalloc_entry_matches_regular_entry_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from imfvideo_b200.ops import cuda as cu

    assert cu.available()
    from imfvideo_b200.ops import kernels as K

    lib = ctypes.CDLL(cu.LIB_PATH)          # the exported symbol, not a Python wrapper
    status = K.status_word(torch.device("cuda", 0))
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for seed, (B, L, H) in enumerate([(1, 2100, 40), (2, 4000, 24)]):
        assert B * H * math.ceil(L / 384) > sms       # items are split: the scratch is in use
        g = torch.Generator(device="cuda").manual_seed(seed)
        q, k, v = (torch.randn(B, L, H, 64, device="cuda", generator=g).bfloat16() for _ in range(3))
        o_ref, _, lse_ref = K.attn_fwd(q, k, v)
        rc, o, lse = _call_noalloc(lib, q, k, v, status)
        assert rc == 0
        torch.cuda.synchronize()
        K.check_status()
        assert (o.float() - o_ref.float()).abs().max() < 2e-2
        assert ((o.float() - o_ref.float()).norm() / o_ref.float().norm()) < 1e-2
        assert (lse - lse_ref).abs().max() < 1e-3
        if seed == 0:
            # and against the plain fp32 formula (one (batch, head) pair at a time: the score
            # matrix of the whole problem would not be small)
            from imfvideo_b200.ops import reference as ref

            for h in (0, H // 2, H - 1):
                ro = ref.attention(q[:, :, h:h + 1].float(), k[:, :, h:h + 1].float(),
                                   v[:, :, h:h + 1].float())
                assert (o[:, :, h:h + 1].float() - ro).abs().max() < 2e-2
                assert ((o[:, :, h:h + 1].float() - ro).norm() / ro.norm()) < 1e-2


def test_noalloc_entry_rejects_oversize_request():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from imfvideo_b200.ops import cuda as cu

    assert cu.available()
    from imfvideo_b200.ops import kernels as K

    lib = ctypes.CDLL(cu.LIB_PATH)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    q = torch.zeros(1, 64, 1, 64, dtype=torch.bfloat16, device="cuda")
    status = K.status_word(torch.device("cuda", 0))
    # wrong head_dim is refused before anything is launched
    bad = torch.zeros(1, 64, 1, 32, dtype=torch.bfloat16, device="cuda")
    rc, _, _ = _call_noalloc(lib, bad, bad, bad, status)
    assert rc == -1
    if sms <= 160:
        pytest.skip("this GPU never needs more partial slots than the built-in array holds")
    big = torch.zeros(1, 384 * (sms + 1), 1, 64, dtype=torch.bfloat16, device="cuda")
    rc, _, _ = _call_noalloc(lib, big, big, big, status)
    assert rc == -4
