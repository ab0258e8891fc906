"""CPU execution of the step programs: an in-process simulator and a gloo transport.

This is the executable specification of the fused CUDA collective: the same programs
(``schedules.py``), the same codec maths (``codec_ref.py``), the same RNG streams.  It is what
runs under ``world_size=2`` gloo in the CPU tests, and it is the oracle that the GPU kernels
are compared with byte for byte.

Reference counterparts: the ring / butterfly callbacks
(testbed_evaluation/new_comm_hooks/utils.py:78-226) and the pure-PyTorch simulation stack
(simulations_llm/new_comm_hooks/comm_hooks.py) which carries codes as bf16 integers instead
of packed bits.
"""
from __future__ import annotations

import queue
import threading
from typing import Dict, List, Optional, Sequence

import numpy as np

from .. import codec_ref as cr
from ..utils import philox
from . import schedules as sch


class RhtCodecCPU:
    """Rotation codec bound to one (seed, step, bucket): see ``codec_ref``."""

    block = cr.BLOCK

    def __init__(self, bits: int, seed: int, step: int, bucket: int, world: int, rank: int = 0,
                 layout: str = "simt"):
        """`layout`: which lane / register holds which coefficient on the wire ("simt": register
        butterflies, "tc": tensor-core rotation; see ``codec_ref``)."""
        self.bits, self.seed, self.step, self.bucket, self.world = bits, seed, step, bucket, world
        self.rank, self.layout = rank, layout
        self.signs = philox.sign_vector(step, bucket, seed)
        # the RNG stream id mixes the bucket in so that buckets do not share uniforms
        self._tag_base = (bucket & 0xFFFF) << 16

    def message_bytes(self, nblocks: int, block_idx=None) -> int:
        return cr.payload_bytes(nblocks, self.bits)

    def rotate(self, x_blocks: np.ndarray) -> np.ndarray:
        return cr.rotate_fwd(x_blocks, self.signs)

    def encode(self, y: np.ndarray, block_idx: np.ndarray, tag: int) -> np.ndarray:
        return cr.encode_blocks(y, self.bits, block_idx, self._tag_base | tag, self.step, self.seed, self.rank,
                                self.world, self.layout)

    def decode(self, msg: np.ndarray, nblocks: int, block_idx=None) -> np.ndarray:
        return cr.decode_blocks(msg, nblocks, self.bits, self.layout)

    def decode_add(self, msg: np.ndarray, nblocks: int, acc: np.ndarray, block_idx=None) -> np.ndarray:
        return cr.decode_add_blocks(msg, nblocks, self.bits, acc, self.layout)

    def finish(self, y: np.ndarray) -> np.ndarray:
        return cr.rotate_inv(y, self.signs, 1.0 / self.world)


class RhtMixCodecCPU(RhtCodecCPU):
    """The rotation codec with a code width per block (`widths`: one entry per block of the bucket)."""

    def __init__(self, widths, seed: int, step: int, bucket: int, world: int, rank: int = 0, layout: str = "simt"):
        super().__init__(8, seed, step, bucket, world, rank, layout)
        self.widths = np.asarray(widths, dtype=np.uint8)
        self.final_scales = {}  # block index -> scale of the all-gathered message (what the next widths derive from)

    def message_bytes(self, nblocks: int, block_idx=None) -> int:
        return cr.mixed_payload_bytes(self.widths[np.asarray(block_idx)])

    def encode(self, y: np.ndarray, block_idx: np.ndarray, tag: int) -> np.ndarray:
        return cr.encode_blocks_mixed(y, self.widths[block_idx], block_idx, self._tag_base | tag, self.step, self.seed,
                                      self.rank, self.world, self.layout)

    def decode(self, msg: np.ndarray, nblocks: int, block_idx=None) -> np.ndarray:
        w = self.widths[np.asarray(block_idx)]
        _, scale = cr._split_mixed(msg, w)
        for k, b in enumerate(np.asarray(block_idx)):
            self.final_scales[int(b)] = float(scale[k])
        return cr.decode_blocks_mixed(msg, w, self.layout)

    def decode_add(self, msg: np.ndarray, nblocks: int, acc: np.ndarray, block_idx=None) -> np.ndarray:
        return cr.decode_blocks_mixed(msg, self.widths[np.asarray(block_idx)], self.layout, acc)

    def block_absmax(self, nblocks: int) -> np.ndarray:
        """absmax of every block of the reduced bucket, as the scales of the final messages give it."""
        out = np.zeros(nblocks, dtype=np.float32)
        for b, s in self.final_scales.items():
            out[b] = np.float32(s) * np.float32(cr.qmax(int(self.widths[b])))
        return out


class LocalTransport:
    """Mailboxes between threads of one process (one thread per simulated rank)."""

    def __init__(self, world: int, timeout: float = 60.0, drop=None):
        """`drop(src, dst, slot) -> bool` lets a test lose messages; `timeout` bounds every receive."""
        self.boxes: List[Dict[int, "queue.Queue"]] = [dict() for _ in range(world)]
        self.lock = threading.Lock()
        self.sent_bytes = [0] * world
        self.timeout = timeout
        self.drop = drop
        self.log: Dict[tuple, np.ndarray] = {}  # (src, dst, slot) -> message bytes, every message ever sent

    def _box(self, rank: int, slot: int) -> "queue.Queue":
        with self.lock:
            return self.boxes[rank].setdefault(slot, queue.Queue())

    def endpoint(self, rank: int) -> "LocalEndpoint":
        return LocalEndpoint(self, rank)


class LocalEndpoint:
    def __init__(self, t: LocalTransport, rank: int):
        self.t, self.rank = t, rank

    def expect(self, incoming: Dict[int, int], sizes: Dict[int, int]) -> None:
        pass

    def send(self, dst: int, slot: int, msg: np.ndarray) -> None:
        self.t.sent_bytes[self.rank] += msg.nbytes
        with self.t.lock:
            self.t.log[(self.rank, dst, slot)] = msg.copy()
        if self.t.drop is not None and self.t.drop(self.rank, dst, slot):
            return
        self.t._box(dst, slot).put(msg.copy())

    def recv(self, slot: int, timeout: Optional[float] = None) -> np.ndarray:
        try:
            return self.t._box(self.rank, slot).get(timeout=self.t.timeout if timeout is None else timeout)
        except queue.Empty:
            raise TimeoutError(f"rank {self.rank}: no message in slot {slot} within the time budget") from None

    def flush(self) -> None:
        pass


class GlooEndpoint:
    """torch.distributed point-to-point transport; the tag carries (collective id, slot)."""

    def __init__(self, group=None, tag_base: int = 0):
        import torch.distributed as dist

        self.dist, self.group, self.tag_base = dist, group, tag_base
        self.rank = dist.get_rank(group)
        self._recv: Dict[int, tuple] = {}
        self._sends: list = []
        self.sent_bytes = 0

    def expect(self, incoming: Dict[int, int], sizes: Dict[int, int]) -> None:
        import torch

        for slot, src in incoming.items():
            buf = torch.empty(max(sizes[slot], 1), dtype=torch.uint8)
            req = self.dist.irecv(buf, src=src, group=self.group, tag=self.tag_base + slot)
            self._recv[slot] = (buf, req, sizes[slot])

    def send(self, dst: int, slot: int, msg: np.ndarray) -> None:
        import torch

        t = torch.from_numpy(np.ascontiguousarray(msg)) if msg.size else torch.zeros(1, dtype=torch.uint8)
        self.sent_bytes += msg.nbytes
        self._sends.append((self.dist.isend(t, dst=dst, group=self.group, tag=self.tag_base + slot), t))

    def recv(self, slot: int, timeout: float = 60.0) -> np.ndarray:
        buf, req, size = self._recv.pop(slot)
        req.wait()
        return buf.numpy()[:size]

    def flush(self) -> None:
        for req, _ in self._sends:
            req.wait()
        self._sends.clear()


def message_sizes(codec, nblocks: int, world: int, topology: str, rank: int) -> Dict[int, int]:  # noqa: D401
    """{slot: bytes} of every message `rank` receives."""
    sizes = {}
    progs = sch.build_all(world, topology)
    for r, prog in enumerate(progs):
        for st in prog:
            lo, hi = sch.shard_range(nblocks, world, st.shard)
            if st.out == sch.OUT_SEND and st.dst == rank:
                sizes[st.send_slot] = codec.message_bytes(hi - lo, np.arange(lo, hi))
            elif st.out == sch.OUT_FINAL and r != rank:
                sizes[sch.ag_slot(world, topology, st.shard)] = codec.message_bytes(hi - lo, np.arange(lo, hi))
    return sizes


def run_rank(x: np.ndarray, codec, rank: int, world: int, topology: str, ep, correlated: bool = False
             ) -> np.ndarray:
    """Execute `rank`'s program on its flat fp32 gradient `x`; returns the mean estimate."""
    n = x.size
    blocks = cr.to_blocks(x)
    nblocks = blocks.shape[0]
    ep.expect(sch.incoming(world, topology)[rank], message_sizes(codec, nblocks, world, topology, rank))
    for st in sch.build_program(rank, world, topology, correlated):
        lo, hi = sch.shard_range(nblocks, world, st.shard)
        nb = hi - lo
        idx = np.arange(lo, hi)
        if st.out == sch.OUT_DECODE:
            msg = ep.recv(st.recv_slot)
            blocks[lo:hi] = codec.finish(codec.decode(msg, nb, idx))
            continue
        v = blocks[lo:hi] if st.local == sch.LOCAL_WS else codec.rotate(blocks[lo:hi])
        for k in range(st.nrecv):
            v = codec.decode_add(ep.recv(st.recv_slot + k), nb, v, idx)
        if st.out == sch.OUT_STORE:
            blocks[lo:hi] = v
        elif st.out == sch.OUT_SEND:
            ep.send(st.dst, st.send_slot, codec.encode(v, idx, st.tag))
        else:  # OUT_FINAL
            msg = codec.encode(v, idx, st.tag)
            for p in range(world):
                if p != rank:
                    ep.send(p, sch.ag_slot(world, topology, st.shard), msg)
            blocks[lo:hi] = codec.finish(codec.decode(msg, nb, idx))
    ep.flush()
    return blocks.reshape(-1)[:n].copy()


def simulate_allreduce(xs: Sequence[np.ndarray], bits: int, topology: str = "ring", seed: int = 0,
                       step: int = 0, bucket: int = 0, codec_factory=None, return_transport: bool = False,
                       transport: Optional[LocalTransport] = None, correlated: bool = False,
                       layout: str = "simt"):
    """Run all ranks of one collective as threads; returns the per-rank results."""
    world = len(xs)
    transport = transport or LocalTransport(world)
    out: List[Optional[np.ndarray]] = [None] * world
    errs: List[BaseException] = []

    def work(r: int) -> None:
        try:
            codec = (codec_factory(bits, seed, step, bucket, world, r) if codec_factory
                     else RhtCodecCPU(bits, seed, step, bucket, world, r, layout))
            out[r] = run_rank(np.asarray(xs[r], dtype=np.float32), codec, r, world, topology, transport.endpoint(r),
                              correlated)
        except BaseException as e:  # surfaced to the caller below
            errs.append(e)

    threads = [threading.Thread(target=work, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errs:
        raise errs[0]
    return (out, transport) if return_transport else out


def allreduce_gloo(x: np.ndarray, bits: int, topology: str, seed: int, step: int, bucket: int, group=None,
                   codec_factory=None, correlated: bool = False) -> np.ndarray:
    """One compressed all-reduce (mean) of a flat fp32 array over a gloo process group."""
    import torch.distributed as dist

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if world == 1:
        return np.asarray(x, dtype=np.float32).copy()
    codec = (codec_factory or RhtCodecCPU)(bits, seed, step, bucket, world, rank)
    tag_base = ((step & 0xFF) << 16) | ((bucket & 0xFF) << 8)
    return run_rank(np.asarray(x, dtype=np.float32), codec, rank, world, topology, GlooEndpoint(group, tag_base),
                    correlated)
