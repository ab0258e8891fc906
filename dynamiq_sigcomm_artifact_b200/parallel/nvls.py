"""Uncompressed all-reduce through the NVSwitch's in-switch reduction (NVLS).

``NvlsAllreduce`` owns a staging buffer in symmetric memory (``torch.distributed._symmetric_memory``: one
allocation per rank, mapped into every peer, plus a MULTICAST mapping when the box exposes one) and launches
``torch.ops.dq.nvls_allreduce`` - this package's own kernel, csrc/kernels/nvls_allreduce.cu - which sums the
ranks' copies inside the switch with ``multimem.ld_reduce`` and writes the result to every rank with
``multimem.st``.  When the box has no multicast support ``NvlsAllreduce.available`` is False and callers fall
back to the point-to-point identity wire of the fused kernel (``FusedAllreduce`` with codec "cast").

Not for tests in which a rank leaves: a rank that dies while its memory is bound to a multicast object can
fault its peers' GPUs; those tests run on CPU / gloo with ``use_nvls`` off.

The reference has no counterpart (its uncompressed baselines go through the library or its own ring,
testbed_evaluation/new_comm_hooks/comm_hooks.py:175-212).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops as _ops
from ..utils import counters
from .fused import CollectiveTimeout, decode_status

FLAG_BYTES = 4096


class NvlsAllreduce:
    def __init__(self, group=None, max_numel: int = 32 << 20, wire_bits: int = 32, ctas: int = 148,
                 timeout_ms: int = 2000):
        self.ops = _ops.require()
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.ctas = int(ctas)
        self.timeout_ns = int(timeout_ms) * 1_000_000
        self.epoch = 0
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.available = False
        self.reason = ""
        self.stage_bytes = 0
        self._buf = None
        self._hdl = None
        self._status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._alloc(int(max_numel), int(wire_bits))

    def _alloc(self, max_numel: int, wire_bits: int) -> None:
        try:
            import torch.distributed._symmetric_memory as symm_mem
        except Exception as e:  # pragma: no cover - older torch
            self.reason = f"symmetric memory is not available in this torch build ({e})"
            return
        unit = 8 * self.world
        self.stage_bytes = (max_numel + unit - 1) // unit * unit * (wire_bits // 8)
        total = self.stage_bytes + FLAG_BYTES
        try:
            buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            hdl = symm_mem.rendezvous(buf, self.group.group_name if hasattr(self.group, "group_name") else self.group)
        except Exception as e:
            self.reason = f"symmetric-memory rendezvous failed: {type(e).__name__}: {e}"
            return
        if not int(getattr(hdl, "multicast_ptr", 0)):
            self.reason = "this box exposes no NVLink multicast object for the allocation"
            self._buf, self._hdl = buf, hdl
            return
        buf.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # every rank's flags are zero before anyone signals
        self._buf, self._hdl = buf, hdl
        self.available = True
        self.max_numel, self.wire_bits = max_numel, wire_bits

    def fits(self, numel: int, wire_bits: int) -> bool:
        unit = 8 * self.world
        return self.available and (numel + unit - 1) // unit * unit * (wire_bits // 8) <= self.stage_bytes

    def allreduce_(self, bucket: torch.Tensor, wire_bits: int = 32, post_scale: Optional[float] = None,
                   ctas: Optional[int] = None) -> torch.Tensor:
        """In-place mean (or `post_scale` x sum) of a flat fp32 / bf16 CUDA tensor on the current stream."""
        if not self.fits(bucket.numel(), wire_bits):
            raise RuntimeError(f"NVLS all-reduce unavailable for {bucket.numel()} elements: {self.reason or 'too large'}")
        flags = [int(p) + self.stage_bytes for p in self._hdl.buffer_ptrs]
        self.epoch += 2
        self.ops.nvls_allreduce(bucket, int(self._hdl.buffer_ptrs[self.rank]), int(self._hdl.multicast_ptr), flags,
                                self.stage_bytes, self._status.data_ptr(), self.rank, self.world, wire_bits,
                                self.epoch, (1.0 / self.world) if post_scale is None else float(post_scale),
                                self.timeout_ns, int(ctas or self.ctas))
        counters.add("nvls_allreduce")
        return bucket

    def check(self) -> None:
        msg = decode_status(self._status.cpu().tolist())
        if msg is not None:
            self._status.zero_()
            raise CollectiveTimeout(f"rank {self.rank}: NVLS all-reduce: {msg}")

    def close(self) -> None:
        self._hdl = None
        self._buf = None
        self.available = False
