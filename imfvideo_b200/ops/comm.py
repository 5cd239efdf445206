"""NVLink-side collectives served by this library's own kernels over peer
memory (``csrc/comm.cu``): reduce-scatter-mean of the owner-major gradient
buffer and all-gather of the orthogonalised updates.

``try_create`` returns ``None`` when peer memory cannot be set up (single GPU,
no P2P, symmetric memory unavailable); callers then use ``torch.distributed``.
"""

from __future__ import annotations

from typing import Optional

import torch


def try_create(world: int, rank: int, device: torch.device, total: int, seg_pad: int):
    try:
        from .comm_impl import PeerComm
    except Exception:
        return None
    try:
        return PeerComm(world, rank, device, total, seg_pad)
    except Exception as exc:      # fall back loudly, once
        if rank == 0:
            print(f"imf_b200: peer-memory collectives unavailable ({type(exc).__name__}: {exc}); "
                  "using torch.distributed", flush=True)
        return None
