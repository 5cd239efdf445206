"""Where one training step spends its device time: runs a few warm-up steps of a
preset on synthetic latents, records one step with ``torch.profiler`` and prints
the device time per kernel / operator, largest first.

    python -m imfvideo_b200.utils.step_profile --preset d256
    python -m imfvideo_b200.utils.step_profile --preset d256_sla2 --top 30
    python -m imfvideo_b200.utils.step_profile --preset d1024 optim.ns_cuda_graph=true
    python -m imfvideo_b200.utils.step_profile --preset d256 --gaps 15     # longest idle gaps
    python -m imfvideo_b200.utils.step_profile --preset d256 --ops 40      # launches per torch op

Times taken under the profiler are for comparing shares, not for quoting a step
time (use ``bench.py`` for that).  The reference has no profiling entry point
(only wall-clock prints in its train loop, reference train.py); this one is an
addition.
"""

from __future__ import annotations

import argparse
from typing import List, Tuple

import torch


def idle_gaps(prof, top: int):
    """The ``top`` longest intervals in which the device ran no kernel, from a profiler
    record: [(gap_us, kernel before, kernel after)], plus the total idle time between the
    first and the last kernel.  Kernels of all streams count as 'busy'."""
    spans = []
    for e in prof.events():
        if e.device_type == torch.autograd.DeviceType.CUDA and e.time_range is not None:
            spans.append((e.time_range.start, e.time_range.end, e.name))
    spans.sort()
    gaps, busy_until, last, idle = [], None, "", 0.0
    for st, en, name in spans:
        if busy_until is not None and st > busy_until:
            gaps.append((st - busy_until, last, name))
            idle += st - busy_until
        if busy_until is None or en > busy_until:
            busy_until, last = en, name
    gaps.sort(reverse=True)
    return gaps[:top], idle


def launch_counts(prof, top: int):
    """Which framework ops launch the most kernels: [(launches, device_us, op name, input
    shapes)], most launches first.  Only kernels launched from inside a torch op are
    attributed (this library's own launches go through ctypes and belong to no op); the
    profile must have been recorded with ``record_shapes=True`` for the shapes to show."""
    acc = {}
    for e in prof.events():
        ks = getattr(e, "kernels", None)
        if e.device_type != torch.autograd.DeviceType.CPU or not ks:
            continue
        key = (e.name, str(getattr(e, "input_shapes", "")))
        c = acc.setdefault(key, [0, 0.0])
        c[0] += len(ks)
        c[1] += sum(k.duration for k in ks)
    rows = [(n, us, name, shapes) for (name, shapes), (n, us) in acc.items()]
    rows.sort(key=lambda r: (-r[0], -r[1], r[2]))
    return rows[:top]


def profile_step(cfg, warmup: int = 2, device: int = 0, gaps: int = 0, ops: int = 0):
    """Returns (rows, step_wall_ms): rows = [(device_us, count, name)], largest first, for one
    training step after ``warmup`` un-profiled steps.  With ``gaps`` > 0 a third value: the
    result of ``idle_gaps``; with ``ops`` > 0 one more: the result of ``launch_counts``."""
    from torch.profiler import ProfilerActivity, profile

    from ..train import Trainer

    cfg.optim.warmup_steps = 0
    tr = Trainer(cfg, device=torch.device("cuda", device), verbose=False)
    x = torch.randn(1, cfg.model.in_channels,
                    cfg.data.latent_frames, *cfg.data.latent_size, device="cuda")
    y = torch.randint(0, 1000, (1,), device="cuda")
    for _ in range(warmup):
        tr.train_step(x, y)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA],
                 record_shapes=ops > 0) as prof:
        a.record()
        tr.train_step(x, y)
        b.record()
        torch.cuda.synchronize()
    rows: List[Tuple[float, int, str]] = []
    for e in prof.key_averages():
        if (e.self_device_time_total > 0 and e.device_type == torch.autograd.DeviceType.CUDA
                and not e.key.startswith("Optimizer.step")):      # a span, not a kernel
            rows.append((e.self_device_time_total, e.count, e.key))
    rows.sort(reverse=True)
    out = [rows, a.elapsed_time(b)]
    if gaps > 0:
        out.append(idle_gaps(prof, gaps))
    if ops > 0:
        out.append(launch_counts(prof, ops))
    return tuple(out)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--preset", default="d256")
    ap.add_argument("--top", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--gaps", type=int, default=0,
                    help="also list this many of the longest idle gaps between kernels")
    ap.add_argument("--ops", type=int, default=0,
                    help="also list this many torch ops by the number of kernels they launch")
    ap.add_argument("overrides", nargs="*", help="group.key=value config overrides")
    args = ap.parse_args(argv)
    from ..config import parse_cli, preset

    cfg = preset(args.preset)
    if args.overrides:
        parse_cli(args.overrides, cfg)
    out = profile_step(cfg, args.warmup, gaps=args.gaps, ops=args.ops)
    rows, wall = out[0], out[1]
    total = sum(r[0] for r in rows)
    print(f"preset {args.preset}: step {wall:.1f} ms under the profiler, "
          f"kernels {total / 1000:.1f} ms in {sum(r[1] for r in rows)} launches")
    for us, n, name in rows[:args.top]:
        print(f"{us / 1000:9.2f} ms {100 * us / total:5.1f} %  x{n:<5d} {name[:100]}")
    if args.gaps:
        top, idle = out[2]
        print(f"idle between the first and the last kernel: {idle / 1000:.2f} ms; longest gaps:")
        for g, before, after in top:
            print(f"{g:9.1f} us  after {before[:60]}  before {after[:60]}")
    if args.ops:
        print("torch ops by kernels launched:")
        for n, us, name, shapes in out[-1]:
            print(f"  x{n:<5d} {us / 1000:8.2f} ms  {name}  {shapes[:90]}")


if __name__ == "__main__":
    main()
