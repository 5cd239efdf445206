from .dataset import LatentDataset, build_loader, InfiniteLoader, DevicePrefetcher  # noqa: F401
