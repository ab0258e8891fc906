"""Loader of the native library and thin Python wrappers around its operators.

The library is built in-tree by :mod:`.build` (``_build/dq_native.so``) and exposes its entry
points as ``torch.ops.dq.*``.  On a machine with a GPU a missing library is an error, never a
silent fallback to eager PyTorch: every GPU code path of this package goes through it.
"""
from __future__ import annotations

import threading

import torch

from . import build as _build

_lock = threading.Lock()
_loaded = False


class NativeLibraryMissing(RuntimeError):
    pass


def load(build_if_missing: bool = False) -> bool:
    """Load ``dq_native.so``; returns True when ``torch.ops.dq`` is usable."""
    global _loaded
    with _lock:
        if _loaded:
            return True
        path = _build.lib_path()
        if not path.exists():
            if not build_if_missing:
                return False
            _build.build()
        torch.ops.load_library(str(path))
        _loaded = True
        return True


def require() -> "torch._ops._OpNamespace":
    """``torch.ops.dq`` or a loud failure."""
    if not load():
        raise NativeLibraryMissing(
            f"{_build.lib_path()} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
            "(or `python -m dynamiq_sigcomm_artifact_b200.ops.build`) before using the GPU paths")
    return torch.ops.dq


def available() -> bool:
    return load()
