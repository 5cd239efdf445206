"""Checkpoint save / resume.

File layout matches the reference (``train.py:657-669``): ``out_dir/
step_{step:07d}.pt`` holding ``{"model", "optimizer", "ema", "step",
"config"}`` of tensors, numbers, strings, tuples and dicts only, so it loads
under ``torch.load(weights_only=True)``.  Added here: the write is atomic
(temp file + fsync + rename; a kill in mid-save corrupted a reference run),
an ``extra`` dict carries RNG state, world size, Muon owner map and sampler
position (``Trainer.save`` fills it), and loading is serialised over ranks to bound host memory
(reference ``train.py:500-519``).
"""

from __future__ import annotations

import gc
import os
from typing import Any, Dict, Optional

import torch


def checkpoint_path(out_dir: str, step: int) -> str:
    return os.path.join(out_dir, f"step_{step:07d}.pt")


def save_checkpoint(path: str, model, optimizer, ema, step: int, config_dict: Dict[str, Any],
                    extra: Optional[Dict[str, Any]] = None) -> str:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    payload = {
        "model": model.state_dict(),
        "optimizer": optimizer.state_dict() if optimizer is not None else None,
        "ema": ema.state_dict() if ema is not None else None,
        "step": int(step),
        "config": config_dict,
    }
    if extra:
        payload["extra"] = extra
    tmp = f"{path}.tmp.{os.getpid()}"
    with open(tmp, "wb") as fh:
        torch.save(payload, fh)
        fh.flush()
        os.fsync(fh.fileno())
    os.replace(tmp, path)
    try:
        dfd = os.open(os.path.dirname(os.path.abspath(path)), os.O_RDONLY)
        os.fsync(dfd)
        os.close(dfd)
    except OSError:
        pass
    return path


def latest_checkpoint(out_dir: str) -> Optional[str]:
    """Newest complete checkpoint in ``out_dir`` (temp files are ignored)."""
    if not os.path.isdir(out_dir):
        return None
    names = sorted(n for n in os.listdir(out_dir)
                   if n.startswith("step_") and n.endswith(".pt"))
    return os.path.join(out_dir, names[-1]) if names else None


def load_checkpoint(path: str, model, optimizer=None, ema=None, rank: int = 0, world: int = 1,
                    barrier=None, strict: bool = True) -> Dict[str, Any]:
    """Restore in place; returns {"step", "config", "extra"}.  One rank reads
    at a time.  A truncated / corrupt file raises ``RuntimeError`` naming the
    path (callers may fall back to ``latest_checkpoint`` of an older step)."""
    info: Dict[str, Any] = {}
    for r in range(world):
        if r == rank:
            try:
                ckpt = torch.load(path, map_location="cpu", weights_only=True)
            except Exception as exc:  # zip/pickle errors differ by failure mode
                raise RuntimeError(f"checkpoint {path!r} is unreadable: {exc}") from exc
            model.load_state_dict(ckpt["model"], strict=strict)
            if optimizer is not None and ckpt.get("optimizer") is not None:
                optimizer.load_state_dict(ckpt["optimizer"])
            if ema is not None and ckpt.get("ema") is not None:
                ema.load_state_dict(ckpt["ema"], strict=strict)
            info = {"step": ckpt["step"], "config": ckpt.get("config"),
                    "extra": ckpt.get("extra", {})}
            del ckpt
            gc.collect()
        if world > 1 and barrier is not None:
            barrier()
    return info


def rng_state() -> Dict[str, Any]:
    st = {"cpu": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state()
    return st


def set_rng_state(st: Dict[str, Any]) -> None:
    if "cpu" in st:
        torch.set_rng_state(st["cpu"].cpu().to(torch.uint8))
    if "cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state(st["cuda"].cpu().to(torch.uint8))
