"""Data tooling: parquet rows -> normalised per-video files (CPU)."""
import os

import numpy as np
import pytest
import torch

pa = pytest.importorskip("pyarrow")


def _write_parquet(path, n, shape, seed):
    import pyarrow.parquet as pq

    g = np.random.default_rng(seed)
    lat = [(g.standard_normal(shape) * (1 + c_scale) + 3.0).astype(np.float32)
           for c_scale in g.random(n)]
    tab = pa.table({
        "caption": [f"clip {seed}-{i}" for i in range(n)],
        "vae_latent_bytes": [x.tobytes() for x in lat],
        "vae_latent_shape": [list(shape)] * n,
        "vae_latent_dtype": ["float32"] * n,
    })
    pq.write_table(tab, path)
    return lat


def test_convert_shrinks_normalises_and_feeds_the_dataset(tmp_path):
    from imfvideo_b200.data import prepare_wan_syn as P
    from imfvideo_b200.data.dataset import LatentDataset

    src = tmp_path / "parquet" / "Part_1"
    os.makedirs(src)
    shape = (16, 3, 8, 12)
    a = _write_parquet(str(src / "latents_chunk_0000.parquet"), 3, shape, 1)
    b = _write_parquet(str(src / "latents_chunk_0001.parquet"), 2, shape, 2)
    out = tmp_path / "out"
    info = P.convert(str(tmp_path / "parquet"), str(out), factor=2, mode="pool", verbose=False)
    assert info["videos"] == 5 and info["latent_shape"] == (16, 3, 4, 6)
    files = sorted(f for f in os.listdir(out) if f.endswith(".pt"))
    assert files == [f"video_{i:06d}.pt" for i in range(5)]
    assert not [f for f in os.listdir(out) if f.endswith(".tmp")]
    st = np.load(out / "stats.npz")
    assert st["mean"].shape == (16, 1, 1, 1) and st["std"].shape == (16, 1, 1, 1)
    raw = torch.stack([P.shrink(torch.from_numpy(x), 2, "pool") for x in a + b])
    mean = raw.double().mean(dim=(0, 2, 3, 4)).float()
    std = raw.double().var(dim=(0, 2, 3, 4), unbiased=False).sqrt().float()
    assert np.allclose(st["mean"].reshape(-1), mean.numpy(), atol=1e-5)
    assert np.allclose(st["std"].reshape(-1), std.numpy(), rtol=1e-4)
    d0 = torch.load(out / "video_000000.pt")
    assert d0["label"] == P.caption_label("clip 1-0") and 0 <= d0["label"] < 1000
    want = (raw[0] - mean.view(16, 1, 1, 1)) / std.view(16, 1, 1, 1)
    assert torch.allclose(d0["latent"], want, atol=1e-5)
    allx = torch.stack([torch.load(out / f)["latent"] for f in files])
    assert allx.mean(dim=(0, 2, 3, 4)).abs().max() < 1e-4
    assert (allx.var(dim=(0, 2, 3, 4), unbiased=False) - 1).abs().max() < 1e-3
    from imfvideo_b200.config import Config

    dc = Config().data
    dc.latent_dir, dc.latent_frames, dc.latent_size = str(out), 3, (4, 6)
    ds = LatentDataset(dc, in_channels=16)
    x, y = ds[1]
    assert x.shape == (16, 3, 4, 6) and int(y) == torch.load(out / files[1])["label"]


def test_crop_mode_and_factor_one():
    from imfvideo_b200.data import prepare_wan_syn as P

    x = torch.arange(2 * 1 * 8 * 12, dtype=torch.float32).reshape(2, 1, 8, 12)
    assert torch.equal(P.shrink(x, 1, "pool"), x)
    c = P.shrink(x, 2, "crop")
    assert c.shape == (2, 1, 4, 6) and torch.equal(c, x[:, :, 2:6, 3:9])
    p = P.shrink(x, 2, "pool")
    assert torch.allclose(p, torch.nn.functional.avg_pool3d(x.unsqueeze(0), (1, 2, 2)).squeeze(0))
