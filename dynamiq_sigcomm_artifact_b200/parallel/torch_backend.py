"""Device-agnostic execution of the step programs with codecs written in PyTorch ops.

Covers every method family on both CPU (gloo) and GPU (NCCL point-to-point) without a
dedicated kernel: the reference's superchunk AEE / MEE codec, the identity wires (bf16, fp16,
fp32), MXFP8, FP4 / FP6, THC's integer bins and OmniReduce's dense rows all plug in as a
:class:`TorchCodec`.  It plays the role of the reference's simulation stack
(simulations_llm/new_comm_hooks/*, the NCCL-P2P callbacks of
testbed_evaluation/new_comm_hooks/utils.py:78-226), with packed payloads instead of codes
carried as bf16.  The `rht` family's production path is the fused CUDA kernel
(parallel/fused.py); this module is its portable sibling.

Programs are cut into *rounds*: in a round every rank executes the steps whose inputs were
delivered in earlier rounds, and all messages produced in the round travel in one
``batch_isend_irecv`` (ring: W-1 rounds of one send + one receive; direct: one round of W-1;
all-gather: one round), which keeps NCCL's send/receive ordering symmetric across ranks.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import schedules as sch

_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox4x32_torch(c0, c1, c2, c3, k0: int, k1: int, rounds: int = 10):
    """Philox-4x32 on int64 tensors holding 32-bit words; same bits as utils/philox.py."""
    c0, c1, c2, c3 = torch.broadcast_tensors(*(c.to(torch.int64) & _MASK for c in (c0, c1, c2, c3)))
    k0, k1 = int(k0) & _MASK, int(k1) & _MASK

    def mulhilo(a: int, b: torch.Tensor):
        # 32x32 -> 64 bit product without overflowing int64: split b into 16-bit halves
        lo16, hi16 = b & 0xFFFF, b >> 16
        p_lo = a * lo16  # < 2^48
        p_hi = a * hi16  # < 2^48
        full_lo = (p_lo + ((p_hi & 0xFFFF) << 16))
        lo = full_lo & _MASK
        hi = ((p_hi >> 16) + (full_lo >> 32)) & _MASK
        return hi, lo

    for _ in range(rounds):
        hi0, lo0 = mulhilo(_M0, c0)
        hi1, lo1 = mulhilo(_M1, c2)
        c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
        k0, k1 = (k0 + _W0) & _MASK, (k1 + _W1) & _MASK
    return c0, c1, c2, c3


def uniform_bytes(n: int, stream: int, step: int, seed: int, device, offset: int = 0) -> torch.Tensor:
    """`n` uniform bytes (uint8): element i comes from Philox-4x32-7 counter (i // 16 + offset, 0, stream, step)."""
    ncall = (n + 15) // 16
    idx = torch.arange(offset, offset + ncall, dtype=torch.int64, device=device)
    zero = torch.zeros(1, dtype=torch.int64, device=device)
    w = philox4x32_torch(idx, zero, zero + (stream & _MASK), zero + (step & _MASK), seed & _MASK, (seed >> 32) & _MASK,
                         rounds=7)
    words = torch.stack(w, dim=-1)  # [ncall, 4]
    by = torch.stack([(words >> (8 * k)) & 0xFF for k in range(4)], dim=-1)  # [ncall, 4, 4]
    return by.reshape(-1)[:n].to(torch.uint8)


class TorchCodec:
    """Interface of a codec executed with tensor ops.  `align` is the shard granularity (elements)."""

    align = 1

    def message_bytes(self, numel: int) -> int:
        raise NotImplementedError

    def encode(self, v: torch.Tensor, first: int, tag: int) -> torch.Tensor:
        """fp32 values [numel] (element `first` of the bucket onwards) -> uint8 [message_bytes]."""
        raise NotImplementedError

    def decode(self, msg: torch.Tensor, numel: int) -> torch.Tensor:
        raise NotImplementedError

    # hooks around the collective; identity by default
    def pre(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def post(self, v: torch.Tensor) -> torch.Tensor:
        return v


def plan_rounds(world: int, topology: str) -> List[List[List[sch.Step]]]:
    """rounds[k][rank] = steps that `rank` executes in round k (identical on every rank)."""
    progs = sch.build_all(world, topology)
    pc = [0] * world
    delivered = [set() for _ in range(world)]
    rounds: List[List[List[sch.Step]]] = []
    while any(pc[r] < len(progs[r]) for r in range(world)):
        this: List[List[sch.Step]] = [[] for _ in range(world)]
        new_msgs: List[Tuple[int, int]] = []
        for r in range(world):
            while pc[r] < len(progs[r]):
                st = progs[r][pc[r]]
                if any((st.recv_slot + k) not in delivered[r] for k in range(st.nrecv)):
                    break
                this[r].append(st)
                pc[r] += 1
                if st.out == sch.OUT_SEND:
                    new_msgs.append((st.dst, st.send_slot))
                elif st.out == sch.OUT_FINAL:
                    new_msgs += [(p, st.send_slot) for p in range(world) if p != r]
        if not any(this):
            raise RuntimeError("schedule cannot make progress")
        for dst, slot in new_msgs:
            delivered[dst].add(slot)
        rounds.append(this)
    return rounds


_ROUND_CACHE: Dict[Tuple[int, str], List[List[List[sch.Step]]]] = {}


def allreduce_torch(x: torch.Tensor, codec: TorchCodec, topology: str = "ring", group=None,
                    transmit: bool = True) -> torch.Tensor:
    """Mean all-reduce of a flat fp32 tensor through `codec`; every rank ends with identical bits."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    n = x.numel()
    v = codec.pre(x.reshape(-1).float())
    nv = v.numel()
    per = (nv + world - 1) // world
    per = (per + codec.align - 1) // codec.align * codec.align

    def rng(shard: int) -> Tuple[int, int]:
        lo = min(shard * per, nv)
        return lo, min(lo + per, nv)

    key = (world, topology)
    if key not in _ROUND_CACHE:
        _ROUND_CACHE[key] = plan_rounds(world, topology)
    rounds = _ROUND_CACHE[key]
    inc = sch.incoming(world, topology)
    progs = sch.build_all(world, topology)
    slot_shard: Dict[int, int] = {}
    for r, prog in enumerate(progs):
        for st in prog:
            if st.out == sch.OUT_SEND and st.dst == rank:
                slot_shard[st.send_slot] = st.shard
            elif st.out == sch.OUT_FINAL and r != rank:
                slot_shard[st.send_slot] = st.shard
    inbox: Dict[int, torch.Tensor] = {}
    for k, rnd in enumerate(rounds):
        sends: List[Tuple[int, int, torch.Tensor]] = []
        for st in rnd[rank]:
            lo, hi = rng(st.shard)
            m = hi - lo
            if st.out == sch.OUT_DECODE:
                if m:
                    v[lo:hi] = codec.decode(inbox.pop(st.recv_slot), m)
                continue
            acc = v[lo:hi]
            for j in range(st.nrecv):
                if m:
                    acc = acc + codec.decode(inbox.pop(st.recv_slot + j), m)
            if st.out == sch.OUT_STORE:
                v[lo:hi] = acc
            elif st.out == sch.OUT_SEND:
                if m:
                    sends.append((st.dst, st.send_slot, codec.encode(acc, lo, st.tag)))
            else:
                if m:
                    msg = codec.encode(acc, lo, st.tag)
                    sends += [(p, st.send_slot, msg) for p in range(world) if p != rank]
                    v[lo:hi] = codec.decode(msg, m)
        # messages that reach this rank in round k: produced by steps of round k on other ranks
        recvs: List[Tuple[int, int, torch.Tensor]] = []
        for r in range(world):
            if r == rank:
                continue
            for st in rnd[r]:
                lo, hi = rng(st.shard)
                if hi <= lo:
                    continue
                if (st.out == sch.OUT_SEND and st.dst == rank) or st.out == sch.OUT_FINAL:
                    buf = torch.empty(codec.message_bytes(hi - lo), dtype=torch.uint8, device=x.device)
                    recvs.append((r, st.send_slot, buf))
        if transmit and (sends or recvs):
            ops = [dist.P2POp(dist.isend, msg, dst, group=group) for dst, _slot, msg in sorted(sends, key=lambda s: (s[0], s[1]))]
            ops += [dist.P2POp(dist.irecv, buf, src, group=group) for src, _slot, buf in sorted(recvs, key=lambda s: (s[0], s[1]))]
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        for _src, slot, buf in recvs:
            inbox[slot] = buf if transmit else torch.zeros_like(buf)
    out = codec.post(v)[:n] / world
    return out
