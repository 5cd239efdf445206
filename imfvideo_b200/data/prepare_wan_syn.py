"""Wan-Syn latent chunks -> training files for ``LatentDataset``.

Same job and file formats as the reference's ``prepare_wan_syn.py``
(reference prepare_wan_syn.py:28-237): the HuggingFace dataset
``FastVideo/Wan-Syn_77x448x832_600k`` ships Wan2.1 VAE latents as parquet rows
(``vae_latent_bytes`` / ``vae_latent_shape`` / ``vae_latent_dtype`` /
``caption``); training wants one ``video_XXXXXX.pt`` per clip holding
``{"latent": (16, T, H, W) float32, "label": int}``, normalised per channel
with the statistics of the WHOLE converted set, plus ``stats.npz`` (mean, std
of shape (16, 1, 1, 1)).

    python -m imfvideo_b200.data.prepare_wan_syn download --videos 1000 --out parquet_dir
    python -m imfvideo_b200.data.prepare_wan_syn convert --parquet-dir parquet_dir \
        --out latents_half --factor 2 --mode pool

Differences in how it is done: the first pass streams rows and keeps only
per-channel sums (float64); files are written through a temporary name and
renamed, so an interrupted run never leaves a half-written sample; the second
pass normalises in a thread pool.
"""

from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import time
from typing import Iterator, List, Tuple

import numpy as np
import torch

REPO_ID = "FastVideo/Wan-Syn_77x448x832_600k"
VIDEOS_PER_CHUNK = 8
NUM_LABELS = 1000


def caption_label(caption: str) -> int:
    """Pseudo class of a clip: md5 of its caption modulo 1000."""
    return int(hashlib.md5((caption or "").encode()).hexdigest(), 16) % NUM_LABELS


def shrink(lat: torch.Tensor, factor: int, mode: str) -> torch.Tensor:
    """(C, T, H, W) -> (C, T, H // factor, W // factor): ``pool`` averages
    factor x factor latent cells (whole scene, but latents the VAE decoder never
    saw), ``crop`` keeps the centre crop (true latents, part of the view)."""
    if factor == 1:
        return lat
    c, t, h, w = lat.shape
    if mode == "crop":
        h2, w2 = h // factor, w // factor
        top, left = (h - h2) // 2, (w - w2) // 2
        return lat[:, :, top:top + h2, left:left + w2].contiguous()
    if mode != "pool":
        raise ValueError(f"unknown mode {mode!r}")
    h2, w2 = h // factor, w // factor
    x = lat[:, :, :h2 * factor, :w2 * factor].reshape(c, t, h2, factor, w2, factor)
    return x.mean(dim=(3, 5))


def _atomic_save(obj, path: str) -> None:
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def parquet_files(root: str) -> List[str]:
    return sorted(os.path.join(dp, f) for dp, _, fs in os.walk(root) for f in fs
                  if f.endswith(".parquet"))


def iter_rows(path: str) -> Iterator[Tuple[torch.Tensor, str]]:
    """Yield (latent float32 (C, T, H, W), caption) for every row of one parquet file."""
    import pyarrow.parquet as pq

    tab = pq.read_table(path, columns=["caption", "vae_latent_bytes", "vae_latent_shape",
                                       "vae_latent_dtype"])
    for r in range(tab.num_rows):
        shape = [int(x) for x in tab["vae_latent_shape"][r].as_py()]
        dtype = np.dtype(tab["vae_latent_dtype"][r].as_py())
        buf = tab["vae_latent_bytes"][r].as_py()
        lat = torch.from_numpy(np.frombuffer(buf, dtype=dtype).reshape(shape).copy()).float()
        yield lat, (tab["caption"][r].as_py() or "")


def convert(parquet_dir: str, out: str, factor: int = 2, mode: str = "pool",
            limit_chunks: int = 0, workers: int = 8, verbose: bool = True) -> dict:
    """Parquet rows -> normalised per-video files + ``stats.npz``.  Returns a summary dict."""
    files = parquet_files(parquet_dir)
    if limit_chunks:
        files = files[:limit_chunks]
    if not files:
        raise FileNotFoundError(f"no parquet files under {parquet_dir}")
    os.makedirs(out, exist_ok=True)
    t0 = time.time()
    paths: List[str] = []
    csum = csq = None
    count = 0
    for fi, f in enumerate(files):
        for lat, cap in iter_rows(f):
            lat = shrink(lat, factor, mode)
            if csum is None:
                csum = torch.zeros(lat.shape[0], dtype=torch.float64)
                csq = torch.zeros(lat.shape[0], dtype=torch.float64)
            p = os.path.join(out, f"video_{len(paths):06d}.pt")
            _atomic_save({"latent": lat, "label": caption_label(cap)}, p)
            paths.append(p)
            d = lat.double()
            csum += d.sum(dim=(1, 2, 3))
            csq += (d * d).sum(dim=(1, 2, 3))
            count += lat[0].numel()
        if verbose and ((fi + 1) % 5 == 0 or fi == len(files) - 1):
            print(f"[{fi + 1}/{len(files)}] {len(paths)} videos, {(time.time() - t0) / 60:.1f} min",
                  flush=True)
    C = csum.numel()
    mean = (csum / count).float().reshape(C, 1, 1, 1)
    var = (csq / count).float().reshape(C, 1, 1, 1) - mean ** 2
    std = var.clamp_min(1e-8).sqrt()
    np.savez(os.path.join(out, "stats.npz"), mean=mean.numpy(), std=std.numpy())

    def normalise(p: str) -> None:
        d = torch.load(p, map_location="cpu")
        d["latent"] = (d["latent"] - mean) / std
        _atomic_save(d, p)

    with cf.ThreadPoolExecutor(max_workers=max(1, workers)) as ex:
        list(ex.map(normalise, paths))
    ex0 = torch.load(paths[0], map_location="cpu")["latent"]
    summary = {"videos": len(paths), "latent_shape": tuple(ex0.shape),
               "mean_range": (float(mean.min()), float(mean.max())),
               "std_range": (float(std.min()), float(std.max()))}
    if verbose:
        print(f"done: {summary}", flush=True)
    return summary


def list_chunks() -> List[str]:
    """Parquet paths of the dataset repository, interleaved across its parts so that a
    prefix of the list samples many parts."""
    from huggingface_hub import HfApi

    files = [f for f in HfApi().list_repo_files(REPO_ID, repo_type="dataset")
             if f.endswith(".parquet")]
    by_part = {}
    for f in files:
        by_part.setdefault(f.split("/")[0], []).append(f)
    parts = sorted(by_part, key=lambda p: int(p.split("_")[1]))
    for p in parts:
        by_part[p].sort()
    out, depth = [], 0
    while any(len(by_part[p]) > depth for p in parts):
        out += [by_part[p][depth] for p in parts if len(by_part[p]) > depth]
        depth += 1
    return out


def download(videos: int, out: str, workers: int = 8) -> List[str]:
    """Fetch enough chunks for about ``videos`` clips (resumable; needs network access and
    the ``huggingface_hub`` package)."""
    try:
        from huggingface_hub import hf_hub_download
    except ImportError as exc:      # offline images do not ship it
        raise RuntimeError("download needs the huggingface_hub package and network access") from exc
    need = max(1, -(-videos // VIDEOS_PER_CHUNK))
    want = list_chunks()[:need]
    os.makedirs(out, exist_ok=True)
    with cf.ThreadPoolExecutor(max_workers=workers) as ex:
        return list(ex.map(lambda p: hf_hub_download(REPO_ID, p, repo_type="dataset",
                                                     local_dir=out), want))


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    d = sub.add_parser("download")
    d.add_argument("--videos", type=int, default=1000)
    d.add_argument("--out", default=".cache/wan_syn_parquet")
    d.add_argument("--workers", type=int, default=8)
    c = sub.add_parser("convert")
    c.add_argument("--parquet-dir", default=".cache/wan_syn_parquet")
    c.add_argument("--out", default=".cache/wan_syn_half")
    c.add_argument("--factor", type=int, default=2)
    c.add_argument("--mode", choices=["pool", "crop"], default="pool")
    c.add_argument("--limit-chunks", type=int, default=0)
    c.add_argument("--workers", type=int, default=8)
    args = ap.parse_args(argv)
    if args.cmd == "download":
        download(args.videos, args.out, args.workers)
    else:
        convert(args.parquet_dir, args.out, args.factor, args.mode, args.limit_chunks,
                args.workers)


if __name__ == "__main__":
    main()
