"""Peer-mapped ("symmetric") device buffers for one NVSwitch box.

Every rank allocates the same-sized buffer through the native launcher
(csrc/launcher/symm.cpp), publishes its IPC handle with ``all_gather_object`` and maps all
the others; kernels then address any rank's buffer by pointer.  This replaces the
reference's transport bring-up: RankMeta all-gather, topology validation and the
sender/receiver constructors of ``RingRdmaManager``
(testbed_evaluation/new_comm_hooks/ring_rdma.py:386-494) and ``ButterflyRdmaManager``
(butterfly_rdma.py:115-285).
"""
from __future__ import annotations

import dataclasses
import socket
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import ops as _ops


@dataclasses.dataclass
class RankMeta:
    """What each rank publishes about itself (cf. RankMeta in ring_rdma.py:80-100)."""

    rank: int
    host: str
    device: int
    device_name: str
    handle: bytes


class TopologyError(RuntimeError):
    pass


def p2p_matrix() -> torch.Tensor:
    """[ndev, ndev, 3] int32: (peer access, performance rank, native atomics)."""
    return _ops.require().topology()


def nvlink_summary(device: int) -> dict:
    """NVLink state of one GPU through NVML (read-only); empty when NVML is unavailable."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(device)
        active = 0
        for link in range(18):
            try:
                if pynvml.nvmlDeviceGetNvLinkState(h, link):
                    active += 1
            except pynvml.NVMLError:
                break
        return {"device": device, "name": pynvml.nvmlDeviceGetName(h), "nvlink_active_links": active}
    except Exception:  # NVML missing or refused: the P2P matrix is still checked
        return {}


def validate_metas(metas, device: int, p2p) -> None:
    """Handshake checks before any peer mapping is opened: one host, one GPU per rank, rank order,
    and peer access from `device` to every other rank's GPU (`p2p[i, j, 0]`).  The reference
    validates rank layout and NVLink pairs the same way before it connects
    (testbed_evaluation/new_comm_hooks/ring_rdma.py:144-161, validate_nvlink_pair)."""
    if any(m is None for m in metas):
        raise TopologyError("a rank did not publish its metadata")
    if [m.rank for m in metas] != list(range(len(metas))):
        raise TopologyError(f"rank metadata out of order: {[m.rank for m in metas]}")
    hosts = {m.host for m in metas}
    if len(hosts) != 1:
        raise TopologyError(f"symmetric buffers need all ranks on one host, got {sorted(hosts)}")
    devs = [m.device for m in metas]
    if len(set(devs)) != len(devs):
        raise TopologyError(f"two ranks share a GPU: {devs}")
    if any(len(m.handle) != 64 for m in metas):
        raise TopologyError("malformed IPC handle (expected 64 bytes)")
    for m in metas:
        if m.device != device and not int(p2p[device][m.device][0]):
            raise TopologyError(f"GPU {device} cannot access GPU {m.device} peer-to-peer")


class SymmetricBuffer:
    """One allocation per rank of a group, all of them mapped into this process."""

    def __init__(self, nbytes: int, group=None, device: Optional[int] = None, validate: bool = True):
        self.ops = _ops.require()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.cuda.current_device() if device is None else device
        self.nbytes = int(nbytes)
        self.local_ptr, handle = self.ops.symm_alloc(self.device, self.nbytes)
        meta = RankMeta(self.rank, socket.gethostname(), self.device, torch.cuda.get_device_name(self.device),
                        bytes(handle.numpy().tobytes()))
        metas: List[Optional[RankMeta]] = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(metas, meta, group=group)
        else:
            metas = [meta]
        self.metas = metas
        if validate:
            self._validate()
        self.ptrs: List[int] = []
        for r, m in enumerate(metas):
            if r == self.rank:
                self.ptrs.append(self.local_ptr)
            else:
                h = torch.frombuffer(bytearray(m.handle), dtype=torch.uint8).clone()
                self.ptrs.append(self.ops.symm_open(self.device, h))
        if self.world > 1:
            dist.barrier(group=group)
        self._closed = False

    def _validate(self) -> None:
        validate_metas(self.metas, self.device, p2p_matrix())

    def local(self) -> torch.Tensor:
        """This rank's buffer as a uint8 tensor (no ownership)."""
        return self.ops.wrap_ptr(self.local_ptr, self.nbytes, self.device)

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's.  Collective: a rank frees its allocation only after
        every rank has closed its mapping of it (freeing memory that a peer still has mapped is undefined
        behaviour), hence two barriers.  If a barrier fails (a rank is gone), the local allocation is leaked
        on purpose rather than freed under a possible mapping, and the failure is logged."""
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        collective = self.world > 1 and dist.is_initialized()
        safe_to_free = True
        if collective:
            safe_to_free = self._barrier("before unmapping the peers")
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self.ops.symm_close(p)
        if collective and safe_to_free:
            safe_to_free = self._barrier("before freeing the local allocation")
        if safe_to_free:
            self.ops.symm_free(self.local_ptr)

    def _barrier(self, what: str) -> bool:
        import logging

        try:
            dist.barrier(group=self.group)
            return True
        except Exception as e:  # a peer never arrived: keep going, but say so and do not free
            logging.getLogger(__name__).warning(
                "rank %d: barrier %s failed (%s); the %d-byte symmetric allocation is not freed", self.rank, what,
                e, self.nbytes)
            return False
