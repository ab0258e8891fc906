"""Host side of the fused compressed all-reduce: buffer layout, plans and launches.

``FusedAllreduce`` is the multi-GPU engine used by the DDP hooks: it owns one symmetric
buffer per rank (mailbox slots, flags, status word, tail scratch), builds the step program of
the chosen topology once, and launches ``torch.ops.dq.fused_allreduce`` - one cooperative
kernel per bucket - on the caller's stream.  ``LocalCluster`` runs all ranks of a collective
in one launch on one GPU (each rank's mailbox is an ordinary tensor); the standalone codec
operators and the single-GPU tests are built on it.

Reference counterparts: the ring / butterfly callbacks and their per-tag send/recv buffers
(testbed_evaluation/new_comm_hooks/utils.py:78-226), ``RingRdmaExchange``
(ring_rdma.py:257-383) and the compressor objects' kernel calls
(utils_aggregation.py:369-569).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import ops as _ops
from ..utils import counters
from . import schedules as sch
from .symm import SymmetricBuffer

BLOCK = 1024


class CollectiveTimeout(RuntimeError):
    """A device-side wait ran out of budget; the kernel returned instead of hanging."""


class MailboxOverrun(RuntimeError):
    """A guard zone around the mailbox or flag region of the symmetric buffer was overwritten."""


CANARY_BYTES = 256
CANARY_VALUE = 0xC5


def _align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


CODECS = {"rht": 0, "rht_tc": 1, "sc_aee": 2, "sc_mee": 3, "mx": 4, "cast": 5, "scmix_aee": 6, "scmix_mee": 7,
          "rht_mix": 8}
RHT_CODECS = ("rht", "rht_tc", "rht_mix")  # messages of these carry one fp32 scale per block after the codes


def block_bytes(bits: int, codec: str = "rht") -> int:
    """Bytes of one encoded 1024-element block inside a message (scales of the rht codec excluded)."""
    if codec.startswith("sc_"):
        return 4 * (16 * (2 * bits + 1) + 2)
    if codec.startswith("scmix_"):  # per-superchunk widths: slots are sized for the widest block
        return 4 * (16 * (2 * 8 + 1) + 2)
    if codec == "mx":
        return 128 * bits + 32
    if codec == "rht_mix":  # a width per block: slots are sized for the widest
        return 128 * 8
    return 128 * bits


@dataclasses.dataclass(frozen=True)
class Layout:
    """Geometry of one collective's slots for (numel, world, bits, codec)."""

    numel: int
    world: int
    bits: int
    codec: str = "rht"

    @property
    def nblocks(self) -> int:
        return (self.numel + BLOCK - 1) // BLOCK

    @property
    def blocks_per_shard(self) -> int:
        return sch.shard_blocks(self.nblocks, self.world)

    @property
    def scales_off(self) -> int:
        return _align(self.blocks_per_shard * block_bytes(self.bits, self.codec), 16)

    @property
    def slot_stride(self) -> int:
        scales = 4 * self.blocks_per_shard if self.codec in RHT_CODECS else 0
        return _align(self.scales_off + scales, 256)


def wire_bytes_per_rank(numel: int, world: int, bits: float, codec: str = "rht") -> int:
    """Bytes one rank puts on NVLink in one collective of `numel` elements (each direction): W - 1
    reduce-scatter messages and its own shard to W - 1 peers, whatever the topology.  For the codecs whose
    width varies per block or superchunk, `bits` is the average width the plan was built for."""
    if world <= 1:
        return 0
    lay = Layout(numel, world, 8 if codec in ("rht_mix",) or codec.startswith("scmix_") else int(bits), codec)
    if codec in RHT_CODECS:
        per_block = 128.0 * bits + 4
    elif codec.startswith("scmix_"):
        per_block = 4 * (32.0 * bits + 18)  # four 256-element superchunk records: codes + 16 scales + header
    else:
        per_block = block_bytes(int(bits), codec)
    return int(2 * (world - 1) * lay.blocks_per_shard * per_block)


def uniform_plan(numel: int, bits: int, device) -> torch.Tensor:
    """int32 [2 nblocks + 1] plan of the "rht_mix" codec with every block at `bits`: exclusive prefix sum of the
    widths (message offsets in units of 128 bytes), then the widths."""
    nb = (int(numel) + BLOCK - 1) // BLOCK
    return torch.cat([torch.arange(nb + 1, dtype=torch.int32) * int(bits),
                      torch.full((nb,), int(bits), dtype=torch.int32)]).to(device)


def program_tensor(rank: int, world: int, topology: str, correlated: bool = False) -> torch.Tensor:
    prog = sch.build_program(rank, world, topology, correlated)
    return torch.tensor([s.as_ints() for s in prog], dtype=torch.int32)


def _rotation_flag(rotation: str) -> bool:
    """"simt": fp32 butterflies, bit-exact against the CPU oracle; "tc": tcgen05 / TMEM rotation."""
    if rotation not in ("simt", "tc"):
        raise ValueError("rotation must be 'simt' or 'tc'")
    return rotation == "tc"


_SC_CACHE: Dict[tuple, tuple] = {}


def codec_args(codec: str, bits: int, device) -> tuple:
    """(codec id, lattice_max, c1, c2, lut) as the native operators take them."""
    if codec in ("rht", "rht_tc", "rht_mix", "mx", "cast"):
        return CODECS[codec], 0.0, 0.0, 0.0, None
    if codec.startswith("scmix_"):
        key = (codec, 0, str(device))
        if key not in _SC_CACHE:
            _SC_CACHE[key] = (CODECS[codec], 1.0, 0.0, 0.0, mix_table(codec[6:], device))
        return _SC_CACHE[key]
    key = (codec, bits, str(device))
    if key not in _SC_CACHE:
        from .codecs import SuperchunkCodec, mee_lattice

        c = SuperchunkCodec(bits, codec[3:])
        lut = None
        if codec == "sc_mee":
            lut = mee_lattice(torch.arange(1 << bits, dtype=torch.float32) - c.R, c.eps).to(device).contiguous()
        _SC_CACHE[key] = (CODECS[codec], float(c.lattice_max), float(c.c1), float(c.c2), lut)
    return _SC_CACHE[key]


def mix_table(lattice: str, device) -> torch.Tensor:
    """Constants of the mixed-width superchunk codec as the kernel reads them (csrc/common/sc_codec.cuh):
    lattice_max / c1 / c2 for widths 2, 4, 8 at [0..2] / [4..6] / [8..10], decode levels at 16 / 20 / 36."""
    from .codecs import SuperchunkCodec, mee_lattice

    t = torch.zeros(292, dtype=torch.float32)
    for i, (bits, base) in enumerate(((2, 16), (4, 20), (8, 36))):
        c = SuperchunkCodec(bits, lattice)
        t[i], t[4 + i], t[8 + i] = float(c.lattice_max), float(c.c1), float(c.c2)
        codes = torch.arange(1 << bits, dtype=torch.float32) - c.R
        t[base: base + (1 << bits)] = mee_lattice(codes, c.eps) if lattice == "mee" else codes
    return t.to(device).contiguous()


STATUS_MESSAGES = {1: "timed out waiting for a peer's flag", 2: "malformed step program",
                   3: "a bulk copy into shared memory did not complete",
                   4: "a tensor-core pass did not signal completion",
                   5: "debug mode: a slot index or a block's offset left its slot; the step was not run"}


def decode_status(words: Sequence[int]) -> Optional[str]:
    code = int(words[0])
    if code == 0:
        return None
    step, cta = (int(words[1]) >> 16) & 0xFFFF, int(words[1]) & 0xFFFF
    return f"{STATUS_MESSAGES.get(code, f'error {code}')} (program step {step}, CTA {cta}, slot {int(words[2])})"


class FusedAllreduce:
    """Compressed all-reduce (mean) over NVLink for the ranks of a process group."""

    def __init__(self, group=None, max_numel: int = 32 << 20, ctas: int = 64, threads: int = 256,
                 timeout_ms: int = 2000, validate: bool = True, rotation: str = "simt", max_ctas: Optional[int] = None,
                 prefetch: bool = True, widest: Tuple[int, str] = (32, "cast"), debug: bool = False):
        """`ctas` is the default grid of a collective; a call may ask for any grid up to `max_ctas`
        (every rank must ask for the same one): a bucket that runs under backward wants a small grid,
        the last bucket of a step has the GPU to itself.

        The mailbox is sized for `max_numel` elements on the `widest` wire (bits, codec) the caller will use
        - (32, "cast"), the fp32 identity wire, unless told otherwise; a 5-bit rotation codec needs a sixth
        of that.  A call that needs more grows the buffers (a collective re-allocation), so callers that know
        their largest bucket and codec pass them here and never re-allocate inside a training step.

        `debug`: every region of the symmetric buffer that peers write into (the two slot sets, the flag
        array) is fenced by 256-byte guard zones filled with a pattern; ``check()`` reads them back and
        raises :class:`MailboxOverrun` if a store landed outside its region; and the kernels run in debug
        mode (process-wide switch): before a step touches a mailbox, every CTA checks the step's slot indices
        and the offset and length of every block of its range against the slot - for the plan-driven codecs
        those come from device memory, where no host-side check sees them - and a violation ends the
        collective with a status (``CollectiveTimeout`` names it) instead of a stray store.  With compute-sanitizer not
        available on every machine, this and the byte-exact oracle comparisons are the overrun net."""
        self.debug = bool(debug)
        self.stats_sink: Optional[dict] = None  # a hook state's "stats": gets the bytes every collective puts on the wire
        if self.debug:
            _ops.require().set_debug(True)
        self.ops = _ops.require()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ctas, self.threads = int(ctas), int(threads)
        self.max_ctas = max(int(max_ctas or 0), self.ctas)
        self.prefetch = bool(prefetch)  # False: no staging buffer, half the shared memory per CTA
        self.timeout_ns = int(timeout_ms) * 1_000_000
        self.validate = validate
        self.tensor_rotation = _rotation_flag(rotation)
        self.device = torch.cuda.current_device()
        self.epoch = 0
        self._programs: Dict[tuple, torch.Tensor] = {}
        self.buf: Optional[SymmetricBuffer] = None
        self.max_numel = 0
        self.slot_bytes = 0
        self.allocations = 0  # how many times the symmetric buffers were (re-)allocated
        self.nslots = sch.n_slots(self.world, "ring")  # same count for every topology
        self._alloc(Layout(int(max_numel), self.world, widest[0], widest[1]).slot_stride, int(max_numel))

    # -- buffers ---------------------------------------------------------------------------
    def _alloc(self, slot_bytes: int, max_numel: int) -> None:
        if self.buf is not None:
            self.buf.close()
        self.allocations += 1
        self.max_numel = int(max_numel)
        self.slot_bytes = _align(int(slot_bytes), 256)
        # layout: [set 0][guard][set 1][guard][flags][guard][status][tail scratch]; a set is slots plus one guard
        self.set_bytes = _align(self.nslots * self.slot_bytes, 4096) + 4096  # the last 4 KiB of a set are its guard
        self.flag_words_per_set = self.nslots * self.max_ctas
        self.off_flags = 2 * self.set_bytes
        flag_bytes = _align(2 * self.flag_words_per_set * 4, 4096)
        self.off_status = self.off_flags + flag_bytes + 4096  # guard after the flags
        self.off_tail = self.off_status + 256
        total = self.off_tail + BLOCK * 4
        self.buf = SymmetricBuffer(total, group=self.group, device=self.device, validate=self.validate)
        local = self.buf.local()
        self._status_view = local[self.off_status: self.off_status + 16].view(torch.int32)
        self._guards = [local[self.set_bytes - 4096: self.set_bytes - 4096 + CANARY_BYTES],
                        local[2 * self.set_bytes - 4096: 2 * self.set_bytes - 4096 + CANARY_BYTES],
                        local[self.off_flags + flag_bytes: self.off_flags + flag_bytes + CANARY_BYTES]]
        for g in self._guards:
            g.fill_(CANARY_VALUE)
        if self.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)  # nobody writes into a peer before its guards are in place

    def ensure_capacity(self, numel: int, bits: int = 32, codec: str = "cast") -> None:
        """Grow the symmetric buffers if a message of `numel` elements on the (bits, codec) wire does not fit a
        slot (collective call: every rank must see the same sizes)."""
        need = Layout(int(numel), self.world, bits, codec).slot_stride
        if need > self.slot_bytes:
            self._alloc(max(need, int(self.slot_bytes * 1.5)), max(int(numel), self.max_numel))

    def mailbox_bytes(self) -> int:
        """Bytes of symmetric memory this rank holds (two slot sets, flags, status, tail scratch)."""
        return self.buf.nbytes if self.buf is not None else 0

    def program(self, topology: str, correlated: bool = False) -> torch.Tensor:
        key = (topology, correlated)
        if key not in self._programs:
            self._programs[key] = program_tensor(self.rank, self.world, topology, correlated)
        return self._programs[key]

    # -- the collective --------------------------------------------------------------------
    def allreduce_(self, bucket: torch.Tensor, bits: int, topology: str = "ring", seed: int = 0, step: int = 0,
                   bucket_id: int = 0, no_transmit: bool = False, correlated: bool = False,
                   codec: Optional[str] = None, ctas: Optional[int] = None,
                   plan: Optional[torch.Tensor] = None, post_scale: Optional[float] = None,
                   wire_bits: Optional[float] = None) -> torch.Tensor:
        """In-place mean all-reduce of a flat fp32/bf16 CUDA tensor on the current stream (`post_scale`: the
        factor applied to the sum instead of 1 / world; 1.0 gives the plain sum).  `wire_bits` only feeds the
        byte accounting (`stats_sink["wire_bytes"]`): the average width of a plan-driven codec.

        `codec`: None (the engine's rotation codec), "sc_aee" / "sc_mee" (the hierarchical superchunk
        codec with 2 / 4 / 8-bit codes), "scmix_aee" / "scmix_mee" (the same with a width per superchunk,
        given by `plan` from ``torch.ops.dq.superchunk_plan``; `bits` is ignored), "mx", "cast"."""
        if self.world == 1:
            return bucket
        codec = codec or ("rht_tc" if self.tensor_rotation else "rht")
        self.ensure_capacity(bucket.numel(), bits, codec)
        lay = Layout(bucket.numel(), self.world, bits, codec)
        grid = int(ctas or self.ctas)
        if not 1 <= grid <= self.max_ctas:
            raise ValueError(f"grid of {grid} CTAs outside 1..{self.max_ctas} (flags are allocated for max_ctas)")
        self.epoch += 1
        parity = self.epoch & 1
        mail = [p + parity * self.set_bytes for p in self.buf.ptrs]
        flags = [p + self.off_flags for p in self.buf.ptrs]
        self.ops.fused_allreduce(
            bucket, self.program(topology, correlated), mail, flags, self.set_bytes - 4096, 2 * self.flag_words_per_set, self.nslots,
            self.buf.local_ptr + self.off_status, self.buf.local_ptr + self.off_tail, self.rank, self.world, bits,
            grid, self.threads, lay.blocks_per_shard, lay.slot_stride, lay.scales_off,
            parity * self.flag_words_per_set, self.epoch, seed, step, bucket_id,
            (1.0 / self.world) if post_scale is None else float(post_scale), self.timeout_ns,
            no_transmit, *codec_args(codec, bits, bucket.device), plan, self.prefetch)
        counters.add("fused_allreduce")
        if self.stats_sink is not None and not no_transmit:
            self.stats_sink["wire_bytes"] += wire_bytes_per_rank(bucket.numel(), self.world,
                                                                 bits if wire_bits is None else wire_bits, codec)
        return bucket

    # -- a code width per block (codec "rht_mix") ------------------------------------------
    def uniform_plan(self, numel: int, bits: int) -> torch.Tensor:
        """The plan of a bucket whose blocks all have `bits`-bit codes (what a bucket starts with)."""
        return uniform_plan(numel, bits, torch.device("cuda", self.device))

    def update_widths_(self, plan: torch.Tensor, numel: int, target_bits: float) -> torch.Tensor:
        """After a collective with codec "rht_mix" (same stream): rewrite `plan` in place with the widths the
        next collective of this bucket should use, from the block scales the collective left in this rank's
        all-gather slots.  Every rank computes the same plan; nothing is communicated or read by the host."""
        lay = Layout(int(numel), self.world, 8, "rht_mix")
        parity = self.epoch & 1
        mailbox = self.buf.local()[parity * self.set_bytes: (parity + 1) * self.set_bytes]
        self.ops.rht_widths_update(mailbox, plan, lay.nblocks, lay.blocks_per_shard, lay.slot_stride, lay.scales_off,
                                   sch.ag_slot(self.world, "ring", 0), int(round(float(target_bits) * lay.nblocks)))
        counters.add("rht_widths_update")
        return plan

    def check(self) -> None:
        """Raise :class:`CollectiveTimeout` if any kernel so far gave up on a wait (synchronises)."""
        words = self._status_view.cpu().tolist()
        msg = decode_status(words)
        if msg is not None:
            self._status_view.zero_()
            raise CollectiveTimeout(f"rank {self.rank}: {msg}")
        if self.debug:
            self.check_guards()

    def check_guards(self) -> None:
        """Raise :class:`MailboxOverrun` if a guard zone no longer holds its pattern (synchronises)."""
        names = ("after slot set 0", "after slot set 1", "after the flag array")
        for name, g in zip(names, self._guards):
            if not bool((g == CANARY_VALUE).all()):
                bad = int((g != CANARY_VALUE).nonzero()[0])
                raise MailboxOverrun(f"rank {self.rank}: guard zone {name} overwritten at byte {bad}")

    def state_dict(self) -> dict:
        return {"epoch": self.epoch}

    def close(self) -> None:
        if self.buf is not None:
            self.buf.close()
            self.buf = None
        if self.debug:
            self.ops.set_debug(False)
            self.debug = False


class LocalCluster:
    """All ranks of a collective on one GPU, one cooperative launch (blockIdx.y = rank)."""

    def __init__(self, world: int, max_numel: int, ctas: int = 8, threads: int = 256, device="cuda",
                 timeout_ms: int = 1000, rotation: str = "simt", prefetch: bool = True, debug: Optional[bool] = None):
        """`debug`: True / False switches the kernels' bounds-checking mode on / off for the whole process
        (None leaves it as it is)."""
        self.ops = _ops.require()
        if debug is not None:
            self.ops.set_debug(bool(debug))
        self.prefetch = bool(prefetch)
        self.tensor_rotation = _rotation_flag(rotation)
        self.world, self.ctas, self.threads = world, ctas, threads
        self.device = torch.device(device)
        self.timeout_ns = timeout_ms * 1_000_000
        self.nslots = sch.n_slots(world, "ring")
        worst = Layout(max_numel, world, 32, "cast")
        self.max_numel = max_numel
        self.mailbox_bytes = self.nslots * worst.slot_stride
        self.mail = [torch.zeros(self.mailbox_bytes, dtype=torch.uint8, device=self.device) for _ in range(world)]
        self.flags = [torch.zeros(self.nslots * ctas, dtype=torch.int32, device=self.device) for _ in range(world)]
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.tail_ws = torch.zeros(world, BLOCK, dtype=torch.float32, device=self.device)
        self.epoch = 0

    def run(self, buckets: List[torch.Tensor], programs: torch.Tensor, bits: int, seed: int = 0, step: int = 0,
            bucket_id: int = 0, post_scale: Optional[float] = None, no_transmit: bool = False,
            preset_flags: bool = False, codec: Optional[str] = None, plan: Optional[torch.Tensor] = None) -> None:
        codec = codec or ("rht_tc" if self.tensor_rotation else "rht")
        lay = Layout(buckets[0].numel(), self.world, bits, codec)
        assert buckets[0].numel() <= self.max_numel
        self.epoch += 1
        if preset_flags:
            for f in self.flags:
                f.fill_(self.epoch)
        self.ops.fused_allreduce_local(
            buckets, programs, self.mail, self.flags, self.status, self.tail_ws, self.nslots, bits, self.ctas,
            self.threads, lay.blocks_per_shard, lay.slot_stride, lay.scales_off, 0, self.epoch, seed, step, bucket_id,
            (1.0 / self.world) if post_scale is None else post_scale, self.timeout_ns, no_transmit,
            *codec_args(codec, bits, buckets[0].device), plan, self.prefetch)

    def update_widths_(self, plan: torch.Tensor, numel: int, target_bits: float, rank: int = 0) -> torch.Tensor:
        """`FusedAllreduce.update_widths_` for the emulated rank `rank` (whose mailbox the last run filled)."""
        lay = Layout(int(numel), self.world, 8, "rht_mix")
        self.ops.rht_widths_update(self.mail[rank], plan, lay.nblocks, lay.blocks_per_shard, lay.slot_stride,
                                   lay.scales_off, sch.ag_slot(self.world, "ring", 0),
                                   int(round(float(target_bits) * lay.nblocks)))
        return plan

    def allreduce_(self, buckets: List[torch.Tensor], bits: int, topology: str = "ring", correlated: bool = False,
                   **kw) -> List[torch.Tensor]:
        progs = torch.stack([program_tensor(r, self.world, topology, correlated) for r in range(self.world)])
        self.run(buckets, progs, bits, **kw)
        return buckets

    def check(self) -> None:
        msg = decode_status(self.status.cpu().tolist())
        if msg is not None:
            self.status.zero_()
            raise CollectiveTimeout(msg)

    def slot_bytes(self, rank: int, slot: int, lay: Layout, nblocks: int) -> torch.Tensor:
        """The encoded blocks of one received message as raw bytes [nblocks * block_bytes]."""
        base = slot * lay.slot_stride
        return self.mail[rank][base: base + nblocks * block_bytes(lay.bits, lay.codec)]

    def slot(self, rank: int, slot: int, lay: Layout, nblocks: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """(code words [nblocks, bits, 32] int32, scales [nblocks] fp32) of one received message."""
        base = slot * lay.slot_stride
        codes = self.mail[rank][base: base + nblocks * 128 * lay.bits].view(torch.int32).view(nblocks, lay.bits, 32)
        scales = self.mail[rank][base + lay.scales_off: base + lay.scales_off + 4 * nblocks].view(torch.float32)
        return codes, scales


class RhtCodec:
    """Standalone rotation-codec operators on one GPU (compress / decompress / hop).

    The equivalents of ``eden_utils.scaling_compress / scaling_decompress / scaling_dec_comp``
    (cuda_kernels/src/srrcomp/eden_utils/eden_utils.cpp:133-219) for the `rht` family; each is
    a one-step program of the fused kernel.  Messages are (code words int32 [nb, bits, 32],
    scales fp32 [nb]).
    """

    def __init__(self, bits: int, max_numel: int, seed: int = 0, ctas: int = 32, threads: int = 256, device="cuda",
                 rotation: str = "simt"):
        self.bits, self.seed = bits, seed
        self.cluster = LocalCluster(1, max_numel, ctas=ctas, threads=threads, device=device, rotation=rotation)

    def _prog(self, step: sch.Step) -> torch.Tensor:
        return torch.tensor([[step.as_ints()]], dtype=torch.int32)

    def _put(self, slot: int, msg, lay: Layout) -> None:
        codes, scales = msg
        c, s = self.cluster.slot(0, slot, lay, codes.shape[0])
        c.copy_(codes)
        s.copy_(scales)

    def compress(self, x: torch.Tensor, step: int = 0, bucket_id: int = 0, tag: int = sch.TAG_ENCODE):
        lay = Layout(x.numel(), 1, self.bits)
        work = x.detach().clone().reshape(-1)
        self.cluster.run([work], self._prog(sch.Step(shard=0, out=sch.OUT_SEND, dst=0, send_slot=0, tag=tag)),
                         self.bits, seed=self.seed, step=step, bucket_id=bucket_id)
        c, s = self.cluster.slot(0, 0, lay, lay.nblocks)
        return c.clone(), s.clone()

    def decompress(self, msg, numel: int, step: int = 0, bucket_id: int = 0, post_scale: float = 1.0,
                   dtype=torch.float32) -> torch.Tensor:
        lay = Layout(numel, 1, self.bits)
        self._put(0, msg, lay)
        out = torch.empty(numel, dtype=dtype, device=self.cluster.device)
        self.cluster.run([out], self._prog(sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_DECODE)), self.bits,
                         seed=self.seed, step=step, bucket_id=bucket_id, post_scale=post_scale, preset_flags=True)
        return out

    def dec_comp(self, msg, x_local: torch.Tensor, step: int = 0, bucket_id: int = 0, tag: int = sch.TAG_ENCODE + 1):
        """decode(msg) + rotate(x_local), re-encoded: one ring hop."""
        lay = Layout(x_local.numel(), 1, self.bits)
        self._put(0, msg, lay)
        work = x_local.detach().clone().reshape(-1)
        self.cluster.run([work], self._prog(sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_SEND, dst=0,
                                                     send_slot=1, tag=tag)),
                         self.bits, seed=self.seed, step=step, bucket_id=bucket_id, preset_flags=True)
        c, s = self.cluster.slot(0, 1, lay, lay.nblocks)
        return c.clone(), s.clone()
