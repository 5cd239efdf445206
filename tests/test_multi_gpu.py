"""GPU (>= 2 devices): the peer-memory gradient reduce-scatter / update
all-gather kernels against the NCCL flat all-reduce path, as child processes
(one per GPU), NVLS off."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys, torch
sys.path.insert(0, os.environ["IMF_ROOT"])
import torch.distributed as dist
from imfvideo_b200.config import preset
from imfvideo_b200.parallel import dist as pdist
from imfvideo_b200.train import Trainer
mode = sys.argv[1]
rank, world, local, device = pdist.init_distributed(timeout_s=120)
sla2 = mode.endswith("_sla2")
mode = mode[:-5] if sla2 else mode
cfg = preset("d256_sla2" if sla2 else "d256")
cfg.model.depth, cfg.model.aux_head_depth = 3, 1
cfg.data.latent_frames, cfg.data.latent_size = (8, (16, 32)) if sla2 else (4, (16, 32))
if sla2:
    cfg.model.sla2_topk = 0.25
    cfg.optim.qk_clip_tau = 1e-3           # every head is over the threshold: the clip runs
cfg.optim.warmup_steps = 0
cfg.run.ema_decay = 0.9
cfg.parallel.grad_sync = "fused_p2p" if mode.startswith("fused_p2p") else mode
if mode == "fused_p2p_fp32":
    cfg.parallel.wire_dtype = "float32"
tr = Trainer(cfg, rank, world, device, verbose=False)
if mode.startswith("fused_p2p"):
    assert getattr(tr.grad_sync, "comm", None) is not None, "peer-memory comm not created"
    assert tr.grad_sync.bucketed == (mode == "fused_p2p")
g = torch.Generator().manual_seed(10 + rank)
for s in range(3):
    x = torch.randn(1, 16, cfg.data.latent_frames, 16, 32, generator=g)
    y = torch.randint(0, 1000, (1,), generator=g)
    torch.manual_seed(100 * s + rank)
    st = tr.train_step(x, y)
from imfvideo_b200.ops import kernels
kernels.check_status()
flat = torch.cat([p.detach().reshape(-1).float() for p in tr.net.parameters()] +
                 [p.detach().reshape(-1).float() for p in tr.ema.parameters()])
ref = flat.clone()
dist.broadcast(ref, src=0)
same = bool(torch.equal(flat, ref))
if rank == 0:
    torch.save({"w": flat.cpu(), "gn": st["grad_norm"]}, sys.argv[2])
print(f"rank {rank} replicas_identical={same} loss={st['loss']:.5f} qk={st['qk_hot']}/{st['qk_smax']:.3f}",
      flush=True)
assert same
if sla2:        # the per-head maxima went through the peer-memory MAX kernel and clipped heads
    assert st["qk_hot"] > 0 and st["qk_smax"] > 0
pdist.shutdown()
'''


def _run(mode, out, n=2):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, IMF_ROOT=ROOT, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-c", CHILD, mode, out]
    # torchrun has no -c: write the child to a file
    path = out + ".child.py"
    with open(path, "w") as fh:
        fh.write(CHILD)
    cmd = cmd[:-4] + [path, mode, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return torch.load(out)


def test_peer_memory_collectives_match_nccl(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    b = _run("nccl_flat", str(tmp_path / "b.pt"))
    for mode in ("fused_p2p", "fused_p2p_fp32"):      # bucketed bf16 wire / whole-arena fp32
        a = _run(mode, str(tmp_path / "a.pt"))
        rel = ((a["w"] - b["w"]).norm() / b["w"].norm()).item()
        assert rel < 2e-3, (mode, rel)       # bf16 model: same update up to summation order
        assert abs(a["gn"] - b["gn"]) / b["gn"] < 2e-2, mode
    _run("fused_p2p_sla2", str(tmp_path / "c.pt"))     # SLA2 blocks + QK-clip statistics over ranks
