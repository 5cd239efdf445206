"""Loader and registry for the sm_100a kernel library (``libimf_b200.so``).

The library is built in-tree by ``imfvideo_b200.ops.build`` with plain nvcc
and exposes ``extern "C"`` launchers that take raw device pointers and a
stream, so there is no dependency on torch's C++ ABI.  The Python wrappers
(autograd Functions) live in ``ops/kernels_*.py`` and register themselves
here by feature name.

Policy: on a machine with a GPU, a missing or unloadable library is an error
(``require()``), never a silent fallback; set ``IMF_B200_ALLOW_FALLBACK=1``
to run the pure-torch path on a GPU deliberately (used by parity tests).
"""

from __future__ import annotations

import ctypes
import os
from typing import Callable, Dict, Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
_LIB_ERR: Optional[str] = None
_FEATURES: Dict[str, bool] = {}
_DISABLED: set = set()
_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libimf_b200.so")


def lib() -> Optional[ctypes.CDLL]:
    global _LIB, _LIB_ERR
    if _LIB is None and _LIB_ERR is None:
        try:
            _LIB = ctypes.CDLL(LIB_PATH)
        except OSError as exc:  # not built, or no CUDA runtime
            _LIB_ERR = str(exc)
    return _LIB


def available() -> bool:
    """True when CUDA tensors should be routed to the kernel library."""
    if os.environ.get("IMF_B200_ALLOW_FALLBACK") == "1" and \
            os.environ.get("IMF_B200_FORCE_TORCH") == "1":
        return False
    if not torch.cuda.is_available():
        return False
    if lib() is None:
        if os.environ.get("IMF_B200_ALLOW_FALLBACK") == "1":
            return False
        raise RuntimeError(
            "imfvideo_b200: CUDA device present but the sm_100a kernel library "
            f"failed to load ({_LIB_ERR}); run `python -m imfvideo_b200.ops.build` "
            "or set IMF_B200_ALLOW_FALLBACK=1 to use the slow pure-torch path")
    _register_all()
    return True


def require() -> ctypes.CDLL:
    l = lib()
    if l is None:
        raise RuntimeError(f"libimf_b200.so not loaded: {_LIB_ERR}")
    return l


def has(feature: str) -> bool:
    return _FEATURES.get(feature, False) and feature not in _DISABLED


def disable(*features: str) -> None:
    """Route the named features to the torch path (debugging / parity)."""
    _DISABLED.update(features)


def enable(*features: str) -> None:
    for f in features:
        _DISABLED.discard(f)


_registered = False


def _register_all() -> None:
    global _registered
    if _registered:
        return
    _registered = True
    from . import kernels  # noqa: F401  (fills _FEATURES and the *_dual hooks)


def register(feature: str, **hooks: Callable) -> None:
    _FEATURES[feature] = True
    globals().update(hooks)


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream
