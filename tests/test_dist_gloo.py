"""CPU, gloo, world_size 2: host-side distributed logic (the reference has no
distributed test at all)."""
import os
import socket
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn(fn, world, *args):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, q) + args) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        r, val = q.get(timeout=240)
        res[r] = val
    for p in procs:
        p.join(timeout=60)
    for r, v in res.items():
        if isinstance(v, str) and v.startswith("ERR"):
            raise AssertionError(f"rank {r}: {v}")
    return res


def _entry(fn, rank, world, port, q, *args):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    torch.set_num_threads(2)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        q.put((rank, out))
    except Exception as exc:  # surface the failure in the parent
        import traceback

        q.put((rank, "ERR " + traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _cfg(mode):
    from imfvideo_b200.config import preset

    cfg = preset("tiny")
    cfg.optim.muon_coeff_mode = "jordan"
    cfg.optim.warmup_steps = 0
    cfg.run.ema_decay = 0.0
    cfg.parallel.grad_sync = mode
    cfg.data.batch_size_per_gpu = 1
    return cfg


def _train_rank(rank, world, mode, steps):
    from imfvideo_b200.train import Trainer

    tr = Trainer(_cfg(mode), rank, world, torch.device("cpu"), verbose=False)
    g = torch.Generator().manual_seed(100 + rank)
    stats = []
    versions_moved = True
    for s in range(steps):
        x = torch.randn(1, 16, 4, 16, 16, generator=g)
        y = torch.randint(0, 1000, (1,), generator=g)
        torch.manual_seed(1000 * s + rank)          # loss-internal noise
        v0 = [p._version for p in tr.net.parameters()]
        stats.append(tr.train_step(x, y))
        # owned or not, a parameter that a step rewrote (through the arenas, after the gather
        # of the other ranks' updates) must show it in its version counter on every rank
        versions_moved &= all(p._version > v for p, v in zip(tr.net.parameters(), v0))
    flat = torch.cat([p.detach().reshape(-1) for p in tr.net.parameters()])
    return flat.numpy().tobytes(), [s["grad_norm"] for s in stats], versions_moved


@pytest.mark.parametrize("mode", ["nccl_flat", "fused_p2p"])
def test_replicas_stay_identical_and_modes_agree(mode):
    res = _spawn(_train_rank, 2, mode, 2)
    (w0, gn0, moved0), (w1, gn1, moved1) = res[0], res[1]
    assert w0 == w1, "replicas diverged"
    assert gn0 == gn1
    assert moved0 and moved1, "a step left version counters where they were"
    if mode != "nccl_flat":
        base = _spawn(_train_rank, 2, "nccl_flat", 2)[0][0]
        a = torch.frombuffer(bytearray(w0), dtype=torch.float32)
        b = torch.frombuffer(bytearray(base), dtype=torch.float32)
        assert torch.allclose(a, b, atol=2e-6), "sync mode changed the update"


def _broadcast_rank(rank, world):
    from imfvideo_b200.parallel import dist as pdist

    torch.manual_seed(rank)
    m = torch.nn.Linear(8, 8)
    pdist.broadcast_module(m)
    return torch.cat([p.detach().reshape(-1) for p in m.parameters()]).numpy().tobytes()


def test_broadcast_init():
    res = _spawn(_broadcast_rank, 2)
    assert res[0] == res[1]


def _heartbeat_rank(rank, world):
    from imfvideo_b200.parallel.dist import Heartbeat, RankLostError

    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, period_s=0.05, stale_s=0.6).start()
    time.sleep(0.3)
    hb.check()                       # both alive
    dist.barrier()
    if rank == 1:
        hb.stop()                    # rank 1 "dies" between steps (host-side injection)
        time.sleep(2.0)
        return "stopped"
    t0 = time.time()
    while time.time() - t0 < 5:
        try:
            hb.check()
        except RankLostError as exc:
            return exc.ranks
        time.sleep(0.1)
    return "not detected"


def test_heartbeat_detects_lost_rank():
    res = _spawn(_heartbeat_rank, 2)
    assert res[0] == [1]


def test_gradient_buckets_partition_the_arena():
    """The per-block gradient buckets of the optimizer engine (what each rank reduces for
    itself while backward runs) cover every parameter element exactly once, give every Muon
    matrix to its owner rank and cut AdamW ranges at the shard boundaries -- for any world
    size, built without communication (world = 3 here, single process)."""
    import torch

    from imfvideo_b200.config import preset
    from imfvideo_b200.optim.moonlight import build_moonlight
    from imfvideo_b200.parallel.flat_engine import FlatEngine
    from imfvideo_b200.train import apply_lr_width_groups, build_model

    cfg = preset("tiny")
    cfg.model.attn_res_block_size = 1
    net, _, _ = build_model(cfg)
    opt = build_moonlight(net, lr=1e-3, weight_decay=0.1, coeff_mode="jordan")
    apply_lr_width_groups(opt, net, cfg.model.hidden_size)
    world = 3
    eng = FlatEngine(opt, net, None, rank=1, world=world, mode="nccl_flat_like")
    nblocks = len(net.shared_blocks) + len(net.u_heads) + len(net.v_heads)
    assert len(eng.buckets) == nblocks + 1
    cover = torch.zeros(eng.total, dtype=torch.int32)
    shard = eng.adam_numel // world
    for b in eng.buckets:
        for start, numel, owner in b:
            cover[start:start + numel] += 1
            if start < eng.muon_total:
                assert owner == start // eng.seg_pad            # the whole matrix sits in its owner's segment
                assert (start + numel - 1) // eng.seg_pad == owner
            else:
                assert owner == (start - eng.muon_total) // shard
                assert (start + numel - 1 - eng.muon_total) // shard == owner
    used = torch.zeros(eng.total, dtype=torch.int32)
    for i, (_, p) in enumerate(eng.muon):
        used[eng.muon_off[i]:eng.muon_off[i] + p.numel()] = 1
    for i, (_, p) in enumerate(eng.adam):
        used[eng.adam_off[i]:eng.adam_off[i] + p.numel()] = 1
    assert torch.equal(cover, used)                              # once each, padding untouched
    # the parameters of block k are all in bucket k
    blocks = list(net.shared_blocks) + list(net.u_heads) + list(net.v_heads)
    for k, blk in enumerate(blocks):
        n = sum(p.numel() for p in blk.parameters())
        assert sum(numel for _, numel, _ in eng.buckets[k]) == n


def _train_and_save(rank, world, out_dir):
    from imfvideo_b200.train import Trainer

    cfg = _cfg("fused_p2p")
    cfg.run.out_dir = out_dir
    cfg.run.ema_decay = 0.9
    tr = Trainer(cfg, rank, world, torch.device("cpu"), verbose=False)
    g = torch.Generator().manual_seed(5 + rank)
    for s in range(4):       # the zero-initialised output layers pass no gradient back at first
        x = torch.randn(1, 16, 4, 16, 16, generator=g)
        y = torch.randint(0, 1000, (1,), generator=g)
        torch.manual_seed(77 * s + rank)
        tr.train_step(x, y)
    path = tr.save()                                    # collective; rank 0 writes
    flat = torch.cat([p.detach().reshape(-1) for p in tr.net.parameters()])
    ema = torch.cat([p.detach().reshape(-1) for p in tr.ema.parameters()])
    # after the save every rank holds the gathered optimizer state: momentum by parameter name
    mom = {n: tr.optimizer.state[p]["momentum_buffer"].clone().reshape(-1).numpy().tobytes()
           for n, p in tr.net.named_parameters() if "momentum_buffer" in tr.optimizer.state.get(p, {})}
    return flat.numpy().tobytes(), ema.numpy().tobytes(), path, mom


def test_checkpoint_of_two_ranks_resumes_on_one(tmp_path):
    """Elastic resume: a checkpoint written by an owner-partitioned two-rank job (each rank holds
    the Muon momentum and the AdamW moments of its own share) loads into a single-rank trainer
    with the full state -- weights, EMA, every momentum buffer of either owner -- and training
    goes on."""
    from imfvideo_b200.train import Trainer

    res = _spawn(_train_and_save, 2, str(tmp_path))
    w0, e0, path, mom0 = res[0]
    assert path and os.path.exists(path) and res[1][2] in (None, path)
    assert mom0 == res[1][3]                            # both ranks hold the gathered state
    cfg = _cfg("none")
    cfg.run.out_dir = str(tmp_path)
    cfg.run.ema_decay = 0.9
    tr = Trainer(cfg, 0, 1, torch.device("cpu"), verbose=False)
    tr.load(path)
    assert tr.step == 4
    flat = torch.cat([p.detach().reshape(-1) for p in tr.net.parameters()])
    ema = torch.cat([p.detach().reshape(-1) for p in tr.ema.parameters()])
    assert flat.numpy().tobytes() == w0 and ema.numpy().tobytes() == e0
    n_muon = n_live = 0
    for name, p in tr.net.named_parameters():
        st = tr.optimizer.state.get(p, {})
        if "momentum_buffer" in st:
            buf = st["momentum_buffer"]
            n_muon += 1
            n_live += int(buf.abs().sum() > 0)
            assert buf.reshape(-1).numpy().tobytes() == mom0[name], name
        elif "exp_avg" in st:
            assert float(st["step"]) == 4.0
    assert n_muon == len(mom0) > 0 and n_live == n_muon
    x, y = torch.randn(1, 16, 4, 16, 16), torch.randint(0, 1000, (1,))
    st = tr.train_step(x, y)
    assert st["loss"] == st["loss"] and not st["skipped"] and tr.step == 5


def _load_and_step(rank, world, out_dir, path):
    from imfvideo_b200.train import Trainer

    cfg = _cfg("fused_p2p")
    cfg.run.out_dir = out_dir
    cfg.run.ema_decay = 0.9
    tr = Trainer(cfg, rank, world, torch.device("cpu"), verbose=False)
    tr.load(path)
    before = torch.cat([p.detach().reshape(-1) for p in tr.net.parameters()]).clone()
    g = torch.Generator().manual_seed(9 + rank)
    x = torch.randn(1, 16, 4, 16, 16, generator=g)
    y = torch.randint(0, 1000, (1,), generator=g)
    st = tr.train_step(x, y)
    after = torch.cat([p.detach().reshape(-1) for p in tr.net.parameters()])
    return (before.numpy().tobytes(), after.numpy().tobytes(), tr.step, bool(st["skipped"]))


def test_checkpoint_of_one_rank_resumes_on_two(tmp_path):
    """The other direction: a single-rank checkpoint loads on two ranks, each taking the
    momentum of the matrices it owns; both start from the saved weights and stay identical
    through the next step."""
    from imfvideo_b200.train import Trainer

    cfg = _cfg("none")
    cfg.run.out_dir = str(tmp_path)
    cfg.run.ema_decay = 0.9
    tr = Trainer(cfg, 0, 1, torch.device("cpu"), verbose=False)
    g = torch.Generator().manual_seed(2)
    for _ in range(4):
        tr.train_step(torch.randn(1, 16, 4, 16, 16, generator=g),
                      torch.randint(0, 1000, (1,), generator=g))
    path = tr.save()
    saved = torch.cat([p.detach().reshape(-1) for p in tr.net.parameters()]).numpy().tobytes()
    res = _spawn(_load_and_step, 2, str(tmp_path), path)
    (b0, a0, s0, k0), (b1, a1, s1, k1) = res[0], res[1]
    assert b0 == saved and b1 == saved
    assert a0 == a1 and a0 != saved
    assert s0 == s1 == 5 and not k0 and not k1
