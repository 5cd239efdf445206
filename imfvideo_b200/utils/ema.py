"""Parameter EMA: theta_ema <- decay * theta_ema + (1 - decay) * theta, as one
multi-tensor lerp (the reference loops per parameter, ``train.py:290-298``)."""

from __future__ import annotations

import torch


@torch.no_grad()
def ema_update(ema, model, decay: float) -> None:
    pe = [p for p in ema.parameters()]
    pm = [p.detach().to(q.dtype) if p.dtype != q.dtype else p.detach()
          for p, q in zip(model.parameters(), pe)]
    if pe:
        torch._foreach_lerp_(pe, pm, 1 - decay)
