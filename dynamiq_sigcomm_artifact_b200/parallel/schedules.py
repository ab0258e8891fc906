"""All-reduce schedules as per-rank step programs.

A schedule is a list of :class:`Step` per rank.  The same program drives three executors:
the single-process simulator and the gloo backend (``cpu_backend.py``) and the persistent
CUDA kernel (``csrc/kernels/fused_allreduce.cu``), which walks the program once per CTA.

Shards: the bucket is cut into ``W`` contiguous shards of ``ceil(nblocks / W)`` codec blocks.
Slots: every message of a collective has its own receive slot at the destination rank, so
no slot is reused inside one collective and no credits are needed; reduce-scatter messages
use slots ``0 .. n_rs_slots-1``, the all-gather message of shard ``i`` uses slot
``n_rs_slots + i``.

Topologies
* ``ring``      - the reference's ring: rank r encodes shard r, and at hop s adds its local
  shard ``(r - s) mod W`` to what arrived from the left and re-encodes it for the right
  (testbed_evaluation/new_comm_hooks/utils.py:78-151, ring_rdma.py:607-629).  A value is
  quantised W times.
* ``butterfly`` - the reference's rotated binomial trees, one per shard, in W-1 serial steps
  (``calc_order``, testbed_evaluation/new_comm_hooks/utils.py:44-75; use at :154-226).
  A value is quantised log2(W)+1 times.  W must be a power of two.
* ``direct``    - NVSwitch-native addition: every rank sends shard i straight to rank i,
  which sums all W contributions in one step; two quantisations, two latency phases.

The all-gather is the same for all three: the owner of a reduced shard writes its encoded
bytes into every peer's slot.  On NVSwitch this moves the same bytes per GPU as the
reference's ring all-gather (which only forwards identical bytes, ring_rdma.py:623-629)
and gives bit-identical results in two fewer latency hops per peer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

# local operand of a step
LOCAL_RAW = 0  # bucket tile holds raw gradients: rotate them first
LOCAL_WS = 1  # bucket tile already holds rotated partial sums (butterfly inner nodes)
# what happens to the step's result
OUT_SEND = 0  # encode and write to `dst`'s slot `send_slot`
OUT_STORE = 1  # keep the rotated partial sum in place in the bucket
OUT_FINAL = 2  # owner: encode, write to every peer's all-gather slot, decode locally
OUT_DECODE = 3  # all-gather receive: decode slot -> inverse rotation -> bucket

TOPOLOGIES = ("ring", "butterfly", "direct")


@dataclass(frozen=True)
class Step:
    shard: int
    local: int = LOCAL_RAW
    recv_slot: int = -1  # first receive slot, -1 if the step consumes no message
    nrecv: int = 0  # number of consecutive receive slots summed by this step
    out: int = OUT_SEND
    dst: int = -1
    send_slot: int = -1
    tag: int = 0  # RNG stream of the encode done by this step

    def as_ints(self) -> Tuple[int, ...]:
        return (self.shard, self.local, self.recv_slot, self.nrecv, self.out, self.dst, self.send_slot, self.tag)


STEP_INTS = 8
TAG_ENCODE = 0x100
TAG_FINAL = 0x200
TAG_STRATIFIED = 0x4000  # flag: round with the rank's stratum of a uniform shared by all ranks


def stratify(prog: List["Step"]) -> List["Step"]:
    """Correlated rounding: every reduce-scatter encode of a block draws from one shared uniform
    per value, u_r = ((r + shift) mod W + u0) / W, so that the W rounding errors that meet in the
    sum are negatively correlated (the reference's `correlated` methods load per-rank stratified
    pools, testbed_evaluation/new_comm_hooks/utils_aggregation.py:385-387,
    simulations_llm/gen_correlated_rand.py:37-56).  The owner's final encode stays independent."""
    import dataclasses

    return [dataclasses.replace(st, tag=TAG_ENCODE | TAG_STRATIFIED) if st.out == OUT_SEND else st for st in prog]


def calc_order(rank: int, size: int) -> List[Tuple[int, int, int, int]]:
    """(send_shard, right, recv_shard, left) for each of the W-1 butterfly steps of `rank`.

    Binomial reduction trees rotated by the shard index: pair (0,1),(2,3).. then the
    winners (1,3),(5,7).., then (3,7); at step j shard i moves from ``(a_j + i) % W`` to
    ``(b_j + i) % W``.
    """
    if size & (size - 1):
        raise ValueError("butterfly needs a power-of-two world size")
    pairs: List[Tuple[int, int]] = []
    alive = list(range(size))
    while len(alive) > 1:
        nxt = []
        for i in range(len(alive) // 2):
            pairs.append((alive[2 * i], alive[2 * i + 1]))
            nxt.append(alive[2 * i + 1])
        alive = nxt
    out = []
    for a, b in pairs:
        send_shard = (rank - a) % size  # the i with (a + i) % W == rank
        right = (b + send_shard) % size
        recv_shard = (rank - b) % size  # the i with (b + i) % W == rank
        left = (a + recv_shard) % size
        out.append((send_shard, right, recv_shard, left))
    return out


def n_rs_slots(world: int, topology: str) -> int:
    return max(world - 1, 1)


def ag_slot(world: int, topology: str, shard: int) -> int:
    return n_rs_slots(world, topology) + shard


def n_slots(world: int, topology: str) -> int:
    return n_rs_slots(world, topology) + world


def owner_of(world: int, topology: str, shard: int) -> int:
    """Rank that holds the fully reduced shard before the all-gather."""
    if topology == "direct":
        return shard
    return (shard - 1) % world  # ring and butterfly: rank r ends up owning shard r+1


def build_program(rank: int, world: int, topology: str, correlated: bool = False) -> List[Step]:
    if correlated:
        return stratify(build_program(rank, world, topology))
    W = world
    if topology not in TOPOLOGIES:
        raise ValueError(f"unknown topology {topology!r}")
    if W == 1:
        return [Step(shard=0, out=OUT_FINAL, tag=TAG_FINAL, send_slot=ag_slot(1, topology, 0))]
    steps: List[Step] = []
    if topology == "ring":
        right = (rank + 1) % W
        steps.append(Step(shard=rank, out=OUT_SEND, dst=right, send_slot=0, tag=TAG_ENCODE))
        for s in range(1, W - 1):
            steps.append(Step(shard=(rank - s) % W, recv_slot=s - 1, nrecv=1, out=OUT_SEND, dst=right,
                              send_slot=s, tag=TAG_ENCODE + s))
        own = (rank + 1) % W
        steps.append(Step(shard=own, recv_slot=W - 2, nrecv=1, out=OUT_FINAL, tag=TAG_FINAL,
                          send_slot=ag_slot(W, topology, own)))
    elif topology == "butterfly":
        order = calc_order(rank, W)
        touched = [False] * W
        for j, (s_shard, right, r_shard, _left) in enumerate(order):
            steps.append(Step(shard=s_shard, local=LOCAL_WS if touched[s_shard] else LOCAL_RAW, out=OUT_SEND,
                              dst=right, send_slot=j, tag=TAG_ENCODE + j))
            last = j == len(order) - 1
            steps.append(Step(shard=r_shard, local=LOCAL_WS if touched[r_shard] else LOCAL_RAW, recv_slot=j,
                              nrecv=1, out=OUT_FINAL if last else OUT_STORE, tag=TAG_FINAL if last else 0,
                              send_slot=ag_slot(W, topology, r_shard) if last else -1))
            touched[r_shard] = True
        own = order[-1][2]
    else:  # direct
        for k in range(1, W):
            dst = (rank + k) % W
            # every source rank rounds with its own RNG stream: with a shared stream the W-1 rounding
            # errors of a block would share the term (u - 1/2) and add coherently at the owner
            steps.append(Step(shard=dst, out=OUT_SEND, dst=dst, send_slot=(rank - dst - 1) % W,
                              tag=TAG_ENCODE + rank))
        own = rank
        steps.append(Step(shard=own, recv_slot=0, nrecv=W - 1, out=OUT_FINAL, tag=TAG_FINAL,
                          send_slot=ag_slot(W, topology, own)))
    assert own == [s for s in range(W) if owner_of(W, topology, s) == rank][0]
    # all-gather receives, nearest producer first
    for k in range(1, W):
        shard = (own + k) % W
        steps.append(Step(shard=shard, recv_slot=ag_slot(W, topology, shard), nrecv=1, out=OUT_DECODE))
    return steps


def build_all(world: int, topology: str, correlated: bool = False) -> List[List[Step]]:
    return [build_program(r, world, topology, correlated) for r in range(world)]


def incoming(world: int, topology: str) -> List[Dict[int, int]]:
    """For every rank: {slot: source rank} over all messages it receives in one collective."""
    progs = build_all(world, topology)
    inc: List[Dict[int, int]] = [dict() for _ in range(world)]
    for r, prog in enumerate(progs):
        for st in prog:
            if st.out == OUT_SEND:
                assert st.send_slot not in inc[st.dst], "slot written twice"
                inc[st.dst][st.send_slot] = r
            elif st.out == OUT_FINAL:
                for p in range(world):
                    if p != r:
                        inc[p][ag_slot(world, topology, st.shard)] = r
    return inc


def shard_blocks(nblocks: int, world: int) -> int:
    """Blocks per shard (the last shards may be short or empty)."""
    return (nblocks + world - 1) // world


def shard_range(nblocks: int, world: int, shard: int) -> Tuple[int, int]:
    per = shard_blocks(nblocks, world)
    lo = min(shard * per, nblocks)
    return lo, min(lo + per, nblocks)


def quantisations(world: int, topology: str) -> int:
    """How many times one value is stochastically rounded on its way through the collective."""
    if world == 1:
        return 1
    if topology == "ring":
        return world
    if topology == "direct":
        return 2
    return world.bit_length()  # log2(W) + 1
