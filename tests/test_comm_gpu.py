"""GPU (one device): the peer-memory collectives of ``csrc/comm.cu`` driven with W
"virtual ranks" = W arenas and W flag arrays that all live on this GPU.

The kernels only see pointer tables, so a table whose entries point at local buffers
exercises exactly the code that runs over NVLink.  The launches of different virtual
ranks run one after another on one stream, so they must never wait for each other:
the host pre-sets every flag to the epoch before the first launch (kernels of
different ranks that really wait on one another are never run on one GPU).

Also here: the bounded wait.  A barrier whose peer flag nobody sets must give up after
the configured bound, record status 6, leave the data alone, and leave the context
usable; ``check_status`` turns the word into an exception.
"""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

MAXR = 16


@pytest.fixture(scope="module")
def C():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from imfvideo_b200.ops import cuda as cu

    assert cu.available(), "kernel library must load on a GPU box"
    from imfvideo_b200.ops import comm_impl

    return comm_impl


def _tables(W, total, dtype=torch.float32, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    arenas = [torch.randn(total, device="cuda", generator=g).to(dtype) for _ in range(W)]
    flags = [torch.zeros(4 * MAXR, dtype=torch.int32, device="cuda") for _ in range(W)]
    return arenas, flags


def _ptrs(ts):
    return (ctypes.c_void_p * len(ts))(*[ctypes.c_void_p(t.data_ptr()) for t in ts])


def _preset(flags, W, epoch):
    for f in flags:
        f[:W] = epoch


@pytest.mark.parametrize("W", [2, 4, 8])
def test_reduce_gather_virtual_ranks(C, W):
    K = C.K
    seg_pad, adam = 4096 + 256 * W, 256 * W * 3
    muon_total, total = W * seg_pad, W * seg_pad + adam
    arenas, flags = _tables(W, total)
    ref = torch.stack(arenas).double().mean(0)
    norms = [torch.zeros(MAXR, dtype=torch.float64, device="cuda") for _ in range(W)]
    part = torch.zeros(512, dtype=torch.float64, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = K.status_word(torch.device("cuda", 0))
    ap, fp, npp = _ptrs(arenas), _ptrs(flags), _ptrs(norms)
    _preset(flags, W, 1)
    for r in range(W):
        K._check(C._lib.imf_comm_reduce(ap, fp, None, r, W, seg_pad, muon_total, adam, 1,
                                        K._ptr(status), npp, K._ptr(part), K._ptr(done),
                                        K._stream()), "reduce")
    shard = adam // W
    sq = 0.0
    for r in range(W):
        own = slice(r * seg_pad, (r + 1) * seg_pad)
        sh = slice(muon_total + r * shard, muon_total + (r + 1) * shard)
        assert torch.allclose(arenas[r][own].double(), ref[own], atol=1e-6)
        assert torch.allclose(arenas[r][sh].double(), ref[sh], atol=1e-6)
        sq += float(ref[own].pow(2).sum() + ref[sh].pow(2).sum())
    for r in range(W):            # every rank's slot array holds every rank's share
        assert abs(float(norms[r][:W].sum()) - sq) < 1e-6 * sq
    _preset(flags, W, 2)
    for r in range(W):
        K._check(C._lib.imf_comm_gather(ap, fp, r, W, muon_total, shard, 4, 2, K._ptr(status),
                                        K._stream()), "gather")
    for r in range(W):
        assert torch.allclose(arenas[r][muon_total:].double(), ref[muon_total:], atol=1e-6)
    K.check_status()


@pytest.mark.parametrize("upd_dtype", [torch.bfloat16, torch.float32])
def test_muon_apply_reads_owner_segments(C, upd_dtype):
    import numpy as np

    from imfvideo_b200.parallel.flat_engine import SEG_DTYPE

    K = C.K
    W, seg_pad = 4, 2048
    # two parameters per owner segment, one of them with an odd length (scalar tail path)
    segs, host = [], np.zeros(2 * W, dtype=SEG_DTYPE)
    for r in range(W):
        segs += [(r * seg_pad, 1000), (r * seg_pad + 1000, 517)]
    for i, (st, n) in enumerate(segs):
        host[i] = (st, n, 1.0 - 1e-3 * (i + 1), 0.01 * (i + 1))
    table = torch.from_numpy(host.view(np.uint8).reshape(-1).copy()).cuda()
    upds, flags = _tables(W, W * seg_pad, dtype=upd_dtype, seed=3)
    P0 = torch.randn(W * seg_pad, device="cuda")
    E0 = torch.randn(W * seg_pad, device="cuda")
    clip = torch.tensor([1.0, 0.0], device="cuda")
    status = K.status_word(torch.device("cuda", 0))
    ema_w = 0.25
    want_p, want_e = P0.clone(), E0.clone()
    for i, (st, n) in enumerate(segs):
        u = upds[st // seg_pad][st:st + n].float()          # the OWNER's copy
        a, b = float(host[i]["a"]), float(host[i]["b"])
        want_p[st:st + n] = P0[st:st + n] * a - b * u
        want_e[st:st + n] = E0[st:st + n] + ema_w * (want_p[st:st + n] - E0[st:st + n])
    _preset(flags, W, 1)
    for r in range(W):
        P, E = P0.clone(), E0.clone()
        K._check(C._lib.imf_comm_muon_apply(_ptrs(upds), _ptrs(flags), r, W, seg_pad, K._ptr(P),
                                            K._ptr(E), K._ptr(table), len(segs), 1000, ema_w,
                                            K._ptr(clip), int(upd_dtype == torch.bfloat16), 1,
                                            K._ptr(status), K._stream()), "muon_apply")
        assert torch.allclose(P, want_p, atol=1e-6) and torch.allclose(E, want_e, atol=1e-6)
    # a skipped step changes nothing
    clip[1] = 1.0
    P = P0.clone()
    K._check(C._lib.imf_comm_muon_apply(_ptrs(upds), _ptrs(flags), 0, W, seg_pad, K._ptr(P), None,
                                        K._ptr(table), len(segs), 1000, ema_w, K._ptr(clip),
                                        int(upd_dtype == torch.bfloat16), 1, K._ptr(status),
                                        K._stream()), "muon_apply")
    assert torch.equal(P, P0)
    K.check_status()


def test_bounded_wait_runs_out_and_context_survives(C):
    K = C.K
    W = 2
    arenas, flags = _tables(W, 1024)
    before = arenas[0].clone()
    status = K.status_word(torch.device("cuda", 0))
    status.zero_()
    old = C.set_peer_wait(0.05)                    # 50 ms
    try:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        # rank 0 of a 2-rank table; nobody ever writes rank 1's flag
        K._check(C._lib.imf_comm_barrier(_ptrs(arenas), _ptrs(flags), 0, W, 1, K._ptr(status),
                                         K._stream()), "barrier")
        # a data kernel behind the same kind of wait must not touch its output
        norms = [torch.zeros(MAXR, dtype=torch.float64, device="cuda") for _ in range(W)]
        part = torch.zeros(512, dtype=torch.float64, device="cuda")
        done = torch.zeros(1, dtype=torch.int32, device="cuda")
        K._check(C._lib.imf_comm_reduce(_ptrs(arenas), _ptrs(flags), None, 0, W, 256, 512, 512, 2,
                                        K._ptr(status), _ptrs(norms), K._ptr(part), K._ptr(done),
                                        K._stream()), "reduce")
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert dt < 1.5, f"the wait did not give up within its bound ({dt:.2f} s)"
        assert int(status[0].item()) == 6
        assert torch.equal(arenas[0], before)
        with pytest.raises(RuntimeError, match="peer"):
            K.check_status()
        # the word was cleared and the context still works: a satisfied barrier passes
        _preset(flags, W, 3)
        K._check(C._lib.imf_comm_barrier(_ptrs(arenas), _ptrs(flags), 0, W, 3, K._ptr(status),
                                         K._stream()), "barrier")
        torch.cuda.synchronize()
        K.check_status()
        assert int(flags[1][0].item()) == 3        # rank 0's signal reached the peer's array
    finally:
        C.set_peer_wait(old)


def test_bucketed_bf16_reduce_norm_and_param_gather_virtual_ranks(C):
    """The bucket path end to end on one GPU: pack (publishes the bucket), reduce (own fp32 +
    peers' bf16, rank order), norm finish, sharded parameters gathered with EMA."""
    import numpy as np

    K = C.K
    W, total = 4, 8192
    g = torch.Generator(device="cuda").manual_seed(7)
    G = [torch.randn(total, device="cuda", generator=g) for _ in range(W)]
    G0 = [x.clone() for x in G]
    wire = [torch.zeros(total, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    flags = [torch.zeros(C.FLAG_INTS, dtype=torch.int32, device="cuda") for _ in range(W)]
    # two buckets; ranges with every owner, one of odd length and odd start (scalar path)
    buckets = [[(0, 1024, 0), (1024, 1000, 1), (2024, 1001, 2), (3025, 71, 3)],
               [(4096, 2048, 3), (6144, 1024, 0), (7168, 1024, 1)]]
    rows = [(s, n, o, 0) for b in buckets for s, n, o in b]
    table = torch.from_numpy(np.array(rows, dtype=np.dtype(C.RANGE_DTYPE)).view(np.uint8)
                             .reshape(-1).copy()).cuda()
    rb = np.dtype(C.RANGE_DTYPE).itemsize
    parts = [torch.zeros(len(rows) * C.BUCKET_BX, dtype=torch.float64, device="cuda")
             for _ in range(W)]
    done = torch.zeros(C.MAX_BUCKETS, dtype=torch.int32, device="cuda")
    status = K.status_word(torch.device("cuda", 0))
    fp, wp = _ptrs(flags), _ptrs(wire)
    vp = ctypes.c_void_p
    first = 0
    for b, bk in enumerate(buckets):
        rng = vp(table.data_ptr() + first * rb)
        for r in range(W):          # every rank packs (and publishes) before any rank reduces
            K._check(C._lib.imf_comm_bucket_pack(fp, K._ptr(G[r]), K._ptr(wire[r]), rng, len(bk), r,
                                                 W, b, 1, vp(done.data_ptr() + 4 * b), K._stream()),
                     "pack")
        for r in range(W):
            K._check(C._lib.imf_comm_bucket_reduce(
                fp, wp, K._ptr(G[r]), rng, len(bk), r, W, b, 1, K._ptr(status),
                vp(parts[r].data_ptr() + 8 * first * C.BUCKET_BX), K._stream()), "reduce")
        first += len(bk)
    sq = [0.0] * W
    for s, n, o in [x for b in buckets for x in b]:
        want = G0[o][s:s + n].clone()
        for q in range(W):
            if q != o:
                want += G0[q][s:s + n].bfloat16().float()
        want /= W
        assert torch.allclose(G[o][s:s + n], want, atol=1e-6), (s, n, o)
        for q in range(W):          # the other ranks' copies of the range are untouched
            if q != o:
                assert torch.equal(G[q][s:s + n], G0[q][s:s + n])
        sq[o] += float(G[o][s:s + n].double().pow(2).sum())     # of what the kernel wrote
    norms = [torch.zeros(MAXR, dtype=torch.float64, device="cuda") for _ in range(W)]
    _preset(flags, W, 1)
    for r in range(W):
        K._check(C._lib.imf_comm_norm_finish(fp, _ptrs(norms), K._ptr(parts[r]), len(rows) * C.BUCKET_BX,
                                             r, W, 1, K._ptr(status), K._stream()), "norm_finish")
    for r in range(W):
        for q in range(W):
            assert abs(float(norms[r][q]) - sq[q]) < 1e-9 * max(1.0, sq[q])
    # sharded parameters: rank q's shard of the AdamW slice is authoritative on rank q
    base, shard, ema_w = 4096, 1024, 0.25
    P = [torch.randn(total, device="cuda", generator=g) for _ in range(W)]
    E0 = torch.randn(total, device="cuda", generator=g)
    truth = P[0].clone()
    for q in range(W):
        truth[base + q * shard: base + (q + 1) * shard] = P[q][base + q * shard: base + (q + 1) * shard]
    clip = torch.tensor([1.0, 0.0], device="cuda")
    _preset(flags, W, 2)
    for r in range(W):
        Pr, Er = P[r].clone(), E0.clone()
        ptrs = _ptrs([Pr if q == r else P[q] for q in range(W)])
        K._check(C._lib.imf_comm_param_gather(fp, ptrs, K._ptr(Pr), K._ptr(Er), r, W, base, shard,
                                              ema_w, K._ptr(clip), 2, K._ptr(status), K._stream()),
                 "param_gather")
        assert torch.equal(Pr[base:], truth[base:]) and torch.equal(Pr[:base], P[r][:base])
        own = slice(base + r * shard, base + (r + 1) * shard)
        want_e = E0 + ema_w * (truth - E0)
        want_e[:base] = E0[:base]
        want_e[own] = E0[own]                   # the owner's EMA is updated by its AdamW kernel
        assert torch.allclose(Er, want_e, atol=1e-7)
    K.check_status()


def test_max_reduce_virtual_ranks(C):
    K = C.K
    W, n = 4, 300
    g = torch.Generator(device="cuda").manual_seed(9)
    ins = [torch.randn(n, device="cuda", generator=g) for _ in range(W)]
    ins[2][5] = float("nan")                      # MAX ignores a NaN when another rank is finite
    flags = [torch.zeros(C.FLAG_INTS, dtype=torch.int32, device="cuda") for _ in range(W)]
    status = K.status_word(torch.device("cuda", 0))
    _preset(flags, W, 1)
    want = torch.stack([torch.nan_to_num(x, nan=float("-inf")) for x in ins]).amax(0)
    for r in range(W):
        out = torch.empty(n, device="cuda")
        K._check(C._lib.imf_comm_max(_ptrs(ins), _ptrs(flags), K._ptr(out), n, r, W, 1,
                                     K._ptr(status), K._stream()), "max")
        assert torch.equal(out, want)
    K.check_status()
