"""In-tree build of the native library (sm_100a only).

Reference counterparts: cuda_kernels/setup.py:14-21 (``eden_utils``) and the JIT loader
rdma_comm_compress/ring_allreduce_ext/__init__.py:82-129.  Differences: one library, built
next to the sources so that it travels with the tree; a fixed ``-gencode`` for sm_100a; no
``--use_fast_math`` (the codec must round like its CPU oracle).
"""
from __future__ import annotations

import os
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
BUILD_DIR = PKG / "_build"
LIB_NAME = "dq_native"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17"]


def sources() -> list[str]:
    out = [str(CSRC / "bindings.cpp")]
    out += sorted(str(p) for p in (CSRC / "launcher").glob("*.cpp"))
    out += sorted(str(p) for p in (CSRC / "kernels").glob("*.cu"))
    return out


def lib_path() -> Path:
    return BUILD_DIR / f"{LIB_NAME}.so"


def build(verbose: bool = False) -> Path:
    """Compile (or re-use an up-to-date) ``_build/dq_native.so`` and return its path."""
    from torch.utils import cpp_extension

    BUILD_DIR.mkdir(exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(min(16, os.cpu_count() or 4)))
    cpp_extension.load(
        name=LIB_NAME,
        sources=sources(),
        extra_cflags=CXX_FLAGS,
        extra_cuda_cflags=NVCC_FLAGS,
        extra_include_paths=[str(CSRC)],
        build_directory=str(BUILD_DIR),
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    return lib_path()


if __name__ == "__main__":
    print(build(verbose=True))
