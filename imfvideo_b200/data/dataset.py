"""Latent datasets and the host->device input pipeline.

``LatentDataset`` reads ``.pt`` files ``{"latent": (C, T, H, W) fp32,
"label": int}`` or, with ``latent_dir="synthetic"``, generates N(0, 1)
latents seeded by index (the reference's synthetic branch passes the (H, W)
tuple twice to ``torch.randn`` and raises, ``train.py:71-77``; this one
works).  ``DevicePrefetcher`` stages batches through pinned host memory and
copies them on a side stream so the copy of step k+1 overlaps step k.
"""

from __future__ import annotations

import os
from typing import Iterator, Optional, Tuple

import torch
from torch.utils.data import DataLoader, Dataset, DistributedSampler


class LatentDataset(Dataset):
    def __init__(self, data_cfg, in_channels: int = 16, num_classes: int = 1000,
                 synthetic_len: int = 100_000):
        self.cfg = data_cfg
        self.in_channels, self.num_classes = in_channels, num_classes
        if data_cfg.latent_dir == "synthetic":
            self.files, self.length = None, synthetic_len
        else:
            self.files = sorted(os.path.join(data_cfg.latent_dir, f)
                                for f in os.listdir(data_cfg.latent_dir) if f.endswith(".pt"))
            self.length = len(self.files)

    def __len__(self) -> int:
        return self.length

    def __getitem__(self, idx: int) -> Tuple[torch.Tensor, int]:
        if self.files is None:
            size = self.cfg.latent_size
            h, w = (size, size) if isinstance(size, int) else size
            gen = torch.Generator().manual_seed(int(idx))
            latent = torch.randn(self.in_channels, self.cfg.latent_frames, h, w, generator=gen)
            return latent, int(idx) % self.num_classes
        item = torch.load(self.files[idx], map_location="cpu", weights_only=True)
        return item["latent"].float(), int(item.get("label", 0))


def build_loader(data_cfg, model_cfg, rank: int, world: int, cuda: bool, seed: int = 0):
    ds = LatentDataset(data_cfg, model_cfg.in_channels, model_cfg.num_classes)
    sampler = (DistributedSampler(ds, num_replicas=world, rank=rank, shuffle=True, seed=seed)
               if world > 1 else None)
    loader = DataLoader(ds, batch_size=data_cfg.batch_size_per_gpu, sampler=sampler,
                        shuffle=sampler is None, num_workers=data_cfg.num_workers,
                        pin_memory=data_cfg.pin_memory and cuda, drop_last=True,
                        persistent_workers=data_cfg.num_workers > 0)
    return ds, sampler, loader


class InfiniteLoader:
    """Endless iterator over a DataLoader that advances the sampler epoch.

    ``state()`` / ``restore()`` give the sampler position (epoch, batches already
    handed out in it) that checkpoints carry: after ``restore`` the iterator starts
    the saved epoch and drops the batches that were consumed before the save."""

    def __init__(self, loader, sampler=None, epoch: int = 0):
        self.loader, self.sampler, self.epoch = loader, sampler, epoch
        self._it: Optional[Iterator] = None
        self.batch = 0            # batches handed out in the current epoch
        self._skip = 0

    def __iter__(self):
        return self

    def state(self, prefetched: int = 0):
        """Position as seen by the consumer; ``prefetched`` = batches taken from this
        iterator that the consumer has not used yet (a prefetcher holds one)."""
        epoch, batch = self.epoch, self.batch - prefetched
        if batch < 0:                       # the prefetched batch closed the previous epoch
            epoch, batch = max(0, epoch - 1), max(0, len(self.loader) + batch)
        return {"epoch": epoch, "batch": batch}

    def restore(self, state) -> None:
        self.epoch, self._skip = int(state.get("epoch", 0)), int(state.get("batch", 0))
        self._it, self.batch = None, 0

    def __next__(self):
        if self._it is None:
            if self.sampler is not None:
                self.sampler.set_epoch(self.epoch)
            self._it = iter(self.loader)
            self.batch = 0
            while self._skip > 0:
                self._skip -= 1
                try:
                    next(self._it)
                    self.batch += 1
                except StopIteration:
                    break
        try:
            out = next(self._it)
            self.batch += 1
            return out
        except StopIteration:
            self.epoch += 1
            self._it = None
            return next(self)


class DevicePrefetcher:
    """Pinned staging + side-stream H2D copy, one batch ahead."""

    def __init__(self, it, device: torch.device):
        self.it, self.device = it, device
        self.cuda = device.type == "cuda"
        self.stream = torch.cuda.Stream(device) if self.cuda else None
        self._next = None
        self._preload()

    def _preload(self) -> None:
        try:
            latents, labels = next(self.it)
        except StopIteration:
            self._next = None
            return
        labels = torch.as_tensor(labels)
        if self.cuda:
            if not latents.is_pinned():
                latents = latents.pin_memory()
            with torch.cuda.stream(self.stream):
                self._next = (latents.to(self.device, non_blocking=True),
                              labels.to(self.device, non_blocking=True))
        else:
            self._next = (latents, labels)

    def __iter__(self):
        return self

    def __next__(self):
        if self._next is None:
            raise StopIteration
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
            for t in self._next:
                t.record_stream(torch.cuda.current_stream(self.device))
        out = self._next
        self._preload()
        return out
