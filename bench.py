#!/usr/bin/env python
"""Headline benchmark: latent tokens/s of one full iMF training step
(guidance passes + fused primal/tangent forward + backward + gradient sync +
Moonlight step + QK-clip + EMA) on the d=256, depth-12, 4-head video DiT with
29,120 latent tokens per sample, batch 1 per GPU, bf16 compute with fp32
master weights, synthetic N(0,1) latents and random-init weights.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 \
        --master-addr 127.0.0.1 --master-port 29500 bench.py --gpus 8 ...
    python bench.py --impl reference ...      # unmodified reference build

Prints ONE JSON line on rank 0.  `value` is device-timed (CUDA events, max
over ranks) with inputs already on the device; `e2e` repeats the measurement
through `Trainer.train_step` with a pinned-host -> device copy of the inputs
and a device -> host read of the loss every step.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOKENS = {"d256": 29120, "d256_sla2": 29120, "d1024": 32760, "wan1p3b": 32760,
          "wan1p3b_dense": 32760, "tiny": 256}
PUBLISHED = None      # the reference publishes no B200 tokens/s figure


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the
    timed region runs (read-only queries)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def _dist_env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return int(os.environ.get("RANK", "0")), world, int(os.environ.get("LOCAL_RANK", "0"))


def _max_over_ranks(x: float, device) -> float:
    import torch
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return x


def _barrier_sync(device):
    import torch
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    if device.type == "cuda":
        torch.cuda.synchronize(device)


class L2Flush:
    def __init__(self, device, mb=256):
        import torch

        self.buf = (torch.empty(mb << 20, dtype=torch.uint8, device=device)
                    if device.type == "cuda" else None)

    def __call__(self):
        if self.buf is not None:
            self.buf.fill_(1)


# ------------------------------------------------------------------ ours ---
def run_ours(args):
    import torch

    from imfvideo_b200.config import preset
    from imfvideo_b200.parallel import dist as pdist
    from imfvideo_b200.train import Trainer

    rank, world, local_rank, device = pdist.init_distributed()
    cfg = preset(args.config)
    cfg.run.ema_decay = 0.9999
    cfg.optim.warmup_steps = 0          # non-zero lr from the first step
    if args.grad_sync:
        cfg.parallel.grad_sync = args.grad_sync
    if args.override:
        from imfvideo_b200.config import parse_cli

        parse_cli(args.override, cfg)
    if device.type != "cuda":
        cfg.loss.autocast_bf16 = False
    trainer = Trainer(cfg, rank, world, device, verbose=False)
    launches = None
    if device.type == "cuda":
        from imfvideo_b200.ops import cuda as cu

        cu.available()
        from imfvideo_b200.ops import kernels

        launches = kernels.LAUNCHES
    B = cfg.data.batch_size_per_gpu
    h, w = cfg.data.latent_size
    shape = (B, cfg.model.in_channels, cfg.data.latent_frames, h, w)
    g = torch.Generator().manual_seed(1234 + rank)
    n_host = 4
    host_lat = [torch.randn(shape, generator=g) for _ in range(n_host)]
    host_lab = [torch.randint(0, cfg.model.num_classes, (B,), generator=g) for _ in range(n_host)]
    if device.type == "cuda":
        host_lat = [t.pin_memory() for t in host_lat]
        host_lab = [t.pin_memory() for t in host_lab]
    dev_lat = [t.to(device) for t in host_lat]
    dev_lab = [t.to(device) for t in host_lab]
    flush = L2Flush(device)

    def step_device(i):
        loss, _parts = trainer.micro_step(dev_lat[i % n_host], dev_lab[i % n_host])
        trainer.optimizer_step()
        return loss

    for i in range(args.warmup):
        step_device(i)
    trainer.timer.summary()          # drop the warm-up phases (no-op unless run.profile_phases)
    _barrier_sync(device)
    sampler = ClockSampler(local_rank).start() if device.type == "cuda" and rank == 0 else None
    n0 = launches.count if launches is not None else 0
    if device.type == "cuda":
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    for i in range(args.steps):
        flush()
        step_device(i)
    if device.type == "cuda":
        e1.record()
    _barrier_sync(device)
    wall = time.perf_counter() - t0
    ms = e0.elapsed_time(e1) if device.type == "cuda" else wall * 1e3
    n_launch = (launches.count - n0) if launches is not None else 0
    clocks = sampler.stop() if sampler is not None else None
    ms = _max_over_ranks(ms, device)
    phases = None
    if cfg.run.profile_phases:       # per-phase device time per step, maximum over ranks
        from imfvideo_b200.utils.timers import PhaseTimer

        phases = {k: v / args.steps
                  for k, v in PhaseTimer.reduce_max(trainer.timer.summary()).items()}
    if device.type == "cuda":
        from imfvideo_b200.ops import kernels

        kernels.check_status()

    # end to end: pinned host -> device copy of the inputs and a device -> host
    # read of the loss every step, through the public Trainer.train_step
    _barrier_sync(device)
    t0 = time.perf_counter()
    last = {}
    for i in range(args.steps):
        last = trainer.train_step(host_lat[i % n_host], host_lab[i % n_host])
    trainer.flush_stats()            # the last step's update kernels and their status word
    _barrier_sync(device)
    e2e_ms = _max_over_ranks((time.perf_counter() - t0) * 1e3, device)

    tokens = TOKENS[args.config] * B * world
    value = tokens * args.steps / (ms / 1e3)
    e2e_value = tokens * args.steps / (e2e_ms / 1e3)
    h2d = sum(t.numel() * t.element_size() for t in (host_lat[0], host_lab[0]))
    if rank == 0:
        out = {
            "metric": "latent tokens/sec/box per iMF train step (device-timed, max over ranks)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": (value / PUBLISHED) if PUBLISHED else None,
            "dtype": "bf16" if cfg.loss.autocast_bf16 else "fp32", "data": "synthetic",
            "impl": "ours",
            "config": {"model": f"iMF video DiT {args.config}: d={cfg.model.hidden_size} "
                                f"depth={cfg.model.depth} aux={cfg.model.aux_head_depth} "
                                f"heads={cfg.model.num_heads} attn={cfg.model.attn_impl}",
                       "global_batch": B * world, "seq_len": TOKENS[args.config],
                       "parallelism": f"dp{world}", "grad_sync": cfg.parallel.grad_sync
                       if world > 1 else "none", "optimizer": cfg.optim.optimizer,
                       "l2": "256 MiB buffer written between timed steps (inside the timed "
                             "region); per-step working set is several GB"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 3 * 8 + 8,
                    "loss": last.get("loss")},
            "gpu_launches": n_launch,
        }
        if phases is not None:
            out["phases_ms_max_over_ranks"] = phases
        print(json.dumps(out), flush=True)
    pdist.shutdown()


# ------------------------------------------------------------- reference ---
def run_reference(args):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "train.py")):
        print(json.dumps({"impl": "reference",
                          "unavailable": "baseline/_ref is missing (reference not installed)"}))
        return
    try:
        from baseline.run_reference import run

        run(args, ref_dir, TOKENS, ClockSampler, L2Flush)
    except Exception as exc:      # the arm must exit 0 with a reason
        rank = int(os.environ.get("RANK", "0"))
        if rank == 0:
            msg = f"{type(exc).__name__}: {exc}".replace("\n", " ")[:300]
            print(json.dumps({"impl": "reference", "unavailable": msg}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="d256", choices=sorted(TOKENS))
    ap.add_argument("--grad-sync", default="")
    ap.add_argument("--override", action="append", default=[], metavar="group.key=value",
                    help="config override of the measured arm, e.g. optim.ns_cuda_graph=true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    _rank, world, _lr = _dist_env()
    if args.gpus != world and world == 1 and args.gpus > 1:
        # convenience: re-launch under torchrun when called directly with --gpus N
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", os.environ.get("MASTER_PORT", "29533"), __file__] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
