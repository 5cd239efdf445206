"""Time the peer-memory collectives on N GPUs of one node (one process per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29560 -m imfvideo_b200.ops.profile_comm --numel 400000000

Gradient reduce-scatter-mean (+ squared norm), AdamW-shard gather and the
weight update with the update all-gather fused in, on a synthetic arena of
``--numel`` fp32 elements (9/10 Muon, 1/10 AdamW), CUDA events on every rank,
maximum over ranks.  Reports the bytes each rank pulls over NVLink and the
achieved fraction of the measured peer-copy bandwidth (770 GB/s per direction).
"""

from __future__ import annotations

import argparse
import ctypes
import json

import numpy as np
import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--numel", type=int, default=400_000_000)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args()
    from ..parallel import dist as pdist

    rank, world, local, device = pdist.init_distributed(timeout_s=120)
    from . import comm as comm_mod
    from . import kernels as K

    seg_pad = (int(args.numel * 0.9) // world + 255) // 256 * 256
    muon_total = seg_pad * world
    adam = (args.numel - muon_total + 256 * world - 1) // (256 * world) * (256 * world)
    total = muon_total + adam
    comm = comm_mod.try_create(world, rank, device, total, seg_pad)
    assert comm is not None, "peer-memory collectives unavailable"
    comm.grad_arena.normal_()
    U = comm.update_arena(torch.bfloat16)
    U.normal_()
    P = torch.randn(total, device=device)
    seg_dtype = np.dtype([("start", "<i8"), ("numel", "<i8"), ("a", "<f4"), ("b", "<f4")])
    nseg = 64 * world
    host = np.zeros(nseg, dtype=seg_dtype)
    per = seg_pad // 64 // 4 * 4
    for i in range(nseg):
        host[i] = ((i // 64) * seg_pad + (i % 64) * per, per, 0.999, 0.01)
    segs = torch.from_numpy(host.view(np.uint8).reshape(-1).copy()).to(device)
    clip = torch.tensor([1.0, 0.0], device=device)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        ms = []
        for _ in range(args.iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        t = torch.tensor([float(np.median(ms))], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    t_reduce = timed(comm.reduce_grads)
    t_apply = timed(lambda: comm.apply_muon_updates(P, None, segs, nseg, per, 0.0, clip))
    K.check_status()
    shard = adam // world
    # bytes this rank reads from the other ranks
    b_reduce = (world - 1) * (seg_pad + shard) * 4 + (world - 1) * shard * 4
    b_apply = (world - 1) * 64 * per * 2
    if rank == 0:
        out = {"world": world, "arena_fp32_elems": total,
               "reduce_scatter_gather_ms": t_reduce, "reduce_nvlink_GB": b_reduce / 1e9,
               "reduce_frac_of_link": b_reduce / (t_reduce * 1e6) / args.link_gbs,
               "fused_gather_apply_ms": t_apply, "apply_nvlink_GB": b_apply / 1e9,
               "apply_frac_of_link": b_apply / (t_apply * 1e6) / args.link_gbs}
        print(json.dumps(out), flush=True)
    pdist.shutdown()


if __name__ == "__main__":
    main()
