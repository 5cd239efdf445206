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
    for s in range(steps):
        x = torch.randn(1, 16, 4, 16, 16, generator=g)
        y = torch.randint(0, 1000, (1,), generator=g)
        torch.manual_seed(1000 * s + rank)          # loss-internal noise
        stats.append(tr.train_step(x, y))
    flat = torch.cat([p.detach().reshape(-1) for p in tr.net.parameters()])
    return flat.numpy().tobytes(), [s["grad_norm"] for s in stats]


@pytest.mark.parametrize("mode", ["nccl_flat", "fused_p2p"])
def test_replicas_stay_identical_and_modes_agree(mode):
    res = _spawn(_train_rank, 2, mode, 2)
    (w0, gn0), (w1, gn1) = res[0], res[1]
    assert w0 == w1, "replicas diverged"
    assert gn0 == gn1
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
