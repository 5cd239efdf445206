import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def reference_dir():
    """Directory holding the reference sources (for parity tests), or None."""
    for cand in ("/root/reference", os.path.join(ROOT, "baseline", "_ref")):
        if os.path.exists(os.path.join(cand, "models", "imf_dit_video.py")):
            return cand
    return None


@pytest.fixture(scope="session")
def ref_modules():
    """Import the reference's model / loss / optimizer modules under private
    names (they use top-level names like ``models`` and ``config``)."""
    d = reference_dir()
    if d is None:
        pytest.skip("reference sources not available")
    names = ("models", "models.imf_dit_video", "imf_video", "moonlight", "config", "train")
    saved = {n: sys.modules.pop(n) for n in names if n in sys.modules}
    sys.path.insert(0, d)
    try:
        import importlib

        mods = {name: importlib.import_module(name)
                for name in ("models.imf_dit_video", "imf_video", "moonlight")}
        assert all(os.path.abspath(m.__file__).startswith(os.path.abspath(d)) for m in mods.values())
    finally:
        sys.path.remove(d)
        for n in names:               # leave no reference module behind under a shared name
            sys.modules.pop(n, None)
        sys.modules.update(saved)
    return mods
