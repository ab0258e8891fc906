"""NVTX ranges and profiler capture windows.

The reference marks its ring phases with NVTX behind ``--enable-nvtx``
(rdma_comm_compress/sample_allreduce.py:34-42,435-445), brackets the timed region or one chosen
step with cudaProfilerStart/Stop (sample_allreduce.py:45-58; smoke_test_new_comm_hooks.py:333-350,
``--nsys_profile_step``) and lets its launchers wrap ranks in ``nsys --capture-range=cudaProfilerApi``.
The same three tools live here; all are no-ops unless enabled.
"""
from __future__ import annotations

import contextlib
import os

import torch

_ENABLED = os.environ.get("DQ_NVTX", "0").lower() in ("1", "true", "yes", "on")


def enable(flag: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(flag)


def enabled() -> bool:
    return _ENABLED and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str):
    """``with nvtx_range("rank0.bucket3.allreduce"):`` - a named range when tracing is on."""
    if enabled():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class ProfilerWindow:
    """Calls cudaProfilerStart before step `step` and cudaProfilerStop after it (-1: never)."""

    def __init__(self, step: int = -1):
        self.step, self.active = int(step), False

    def before(self, step: int) -> None:
        if step == self.step and torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            self.active = True

    def after(self, step: int) -> None:
        if self.active and step == self.step:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
            self.active = False
