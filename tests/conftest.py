import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def reference_dir():
    """Directory holding the reference sources (for parity tests), or None: the
    ``IMF_REFERENCE_DIR`` environment variable, a ``reference`` checkout beside this
    repository, or the copy installed for the benchmark's reference arm."""
    cands = [os.environ.get("IMF_REFERENCE_DIR"),
             os.path.join(os.path.dirname(ROOT), "reference"),
             os.path.join(ROOT, "baseline", "_ref")]
    for cand in cands:
        if cand and os.path.exists(os.path.join(cand, "models", "imf_dit_video.py")):
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
