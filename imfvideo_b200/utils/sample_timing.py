"""Time the few-step sampler (``IMFVideoLoss.sample``) of a preset on one GPU.

    python -m imfvideo_b200.utils.sample_timing --preset d256_sla2 --steps 4

The sampler runs the network's u branch under ``no_grad``: the same kernels as training,
primal only (no tangent, no log-sum-exp, bf16 weight copies cached across steps).  Prints
one JSON line: milliseconds per sample (CUDA events, after one warm-up sample).
"""

from __future__ import annotations

import argparse
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="d256")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    from ..config import preset
    from ..train import Trainer

    cfg = preset(args.preset)
    cfg.run.ema_decay = 0.0
    tr = Trainer(cfg, device=torch.device("cuda", 0), verbose=False)
    h, w = cfg.data.latent_size
    z = torch.randn(1, cfg.model.in_channels, cfg.data.latent_frames, h, w, device="cuda")
    y = torch.randint(0, cfg.model.num_classes, (1,), device="cuda")
    tr.net.eval()
    tr.loss_mod.sample(z, y, num_steps=args.steps)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.iters):
        out = tr.loss_mod.sample(z, y, num_steps=args.steps)
    b.record()
    torch.cuda.synchronize()
    from ..ops import kernels

    kernels.check_status()
    print(json.dumps({"preset": args.preset, "sampler_steps": args.steps,
                      "ms_per_sample": a.elapsed_time(b) / args.iters,
                      "finite": bool(torch.isfinite(out).all())}))


if __name__ == "__main__":
    main()
