"""Step programs: coverage, slot uniqueness, reference calc_order, simulator NMSE and determinism."""
import numpy as np
import pytest

from dynamiq_sigcomm_artifact_b200 import codec_ref as cr
from dynamiq_sigcomm_artifact_b200.parallel import cpu_backend as cb
from dynamiq_sigcomm_artifact_b200.parallel import schedules as sch

from helpers import heavy_tail_grad


def _reference_calc_order(rank, size):
    """Restatement of the reference's butterfly order as published in its README tables:
    pairs (0,1),(2,3),...; winners (1,3),(5,7); (3,7) - each rotated by the shard index."""
    pairs, alive = [], list(range(size))
    while len(alive) != 1:
        nxt = []
        for i in range(len(alive) // 2):
            pairs.append([alive[2 * i], alive[2 * i + 1]])
            nxt.append(alive[2 * i + 1])
        alive = nxt
    res = []
    for a, b in pairs:
        row = [None] * 4
        for i in range(size):
            if (a + i) % size == rank:
                row[0], row[1] = i, (b + i) % size
            if (b + i) % size == rank:
                row[2], row[3] = i, (a + i) % size
        res.append(tuple(row))
    return res


@pytest.mark.parametrize("world", [2, 4, 8])
def test_calc_order_matches_reference(world):
    for r in range(world):
        assert sch.calc_order(r, world) == _reference_calc_order(r, world)


@pytest.mark.parametrize("topology", sch.TOPOLOGIES)
@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_every_shard_reduced_once_and_gathered_everywhere(world, topology):
    if topology == "butterfly" and world & (world - 1):
        with pytest.raises(ValueError):
            sch.build_all(world, topology)
        return
    progs = sch.build_all(world, topology)
    inc = sch.incoming(world, topology)  # asserts that no slot is written twice
    # symbolic execution: track which ranks' contributions each message / partial sum holds
    mail = [dict() for _ in range(world)]
    ws = [dict() for _ in range(world)]
    final = [dict() for _ in range(world)]
    pc = [0] * world
    progress = True
    while progress:
        progress = False
        for r in range(world):
            while pc[r] < len(progs[r]):
                st = progs[r][pc[r]]
                need = [st.recv_slot + k for k in range(st.nrecv)]
                if any(s not in mail[r] for s in need):
                    break
                if st.out == sch.OUT_DECODE:
                    shard, contrib = mail[r][st.recv_slot]
                    assert shard == st.shard
                    final[r][st.shard] = contrib
                else:
                    contrib = set(ws[r][st.shard]) if st.local == sch.LOCAL_WS else {r}
                    for s in need:
                        shard, c = mail[r][s]
                        assert shard == st.shard and not (contrib & c), "a contribution was added twice"
                        contrib |= c
                    if st.out == sch.OUT_STORE:
                        ws[r][st.shard] = contrib
                    elif st.out == sch.OUT_SEND:
                        mail[st.dst][st.send_slot] = (st.shard, frozenset(contrib))
                    else:
                        final[r][st.shard] = frozenset(contrib)
                        for p in range(world):
                            if p != r:
                                mail[p][st.send_slot] = (st.shard, frozenset(contrib))
                pc[r] += 1
                progress = True
    assert all(pc[r] == len(progs[r]) for r in range(world)), "schedule deadlocks"
    for r in range(world):
        assert set(inc[r]) == set(mail[r])
        for shard in range(world):
            assert final[r][shard] == frozenset(range(world))
    assert all(len(p) <= 32 for p in progs)


@pytest.mark.parametrize("topology", sch.TOPOLOGIES)
def test_simulated_allreduce_nmse_and_rank_agreement(topology):
    world, n = 4, 10 * 1024 + 100
    xs = [heavy_tail_grad(n, 10 + r) for r in range(world)]
    exact = np.mean(np.stack(xs).astype(np.float64), 0)
    prev = None
    for bits in (4, 5, 8):
        outs = cb.simulate_allreduce(xs, bits, topology, seed=5)
        assert all(np.array_equal(outs[0], o) for o in outs), "ranks disagree"
        e = cr.nmse(outs[0], exact)
        assert e < {4: 0.2, 5: 0.05, 8: 1e-3}[bits]
        assert prev is None or e < prev
        prev = e
    again = cb.simulate_allreduce(xs, 5, topology, seed=5)
    assert np.array_equal(again[0], cb.simulate_allreduce(xs, 5, topology, seed=5)[0])
    other = cb.simulate_allreduce(xs, 5, topology, seed=6)
    assert not np.array_equal(again[0], other[0])


def test_wire_bytes_match_the_schedule():
    world, n, bits = 4, 64 * 1024, 5
    xs = [heavy_tail_grad(n, r) for r in range(world)]
    _, tr = cb.simulate_allreduce(xs, bits, "ring", return_transport=True)
    per_shard = cr.payload_bytes(16, bits)
    assert tr.sent_bytes == [2 * (world - 1) * per_shard] * world


def test_butterfly_requantises_less_than_ring():
    assert sch.quantisations(8, "ring") == 8 and sch.quantisations(8, "butterfly") == 4
    assert sch.quantisations(8, "direct") == 2


def test_direct_sources_round_with_distinct_streams_and_correlated_is_better():
    progs = sch.build_all(4, "direct")
    tags = {(r, st.tag) for r, p in enumerate(progs) for st in p if st.out == sch.OUT_SEND}
    assert len({t for _, t in tags}) == 4  # one RNG stream per source rank
    strat = sch.build_program(1, 4, "ring", correlated=True)
    assert all((st.tag & sch.TAG_STRATIFIED) for st in strat if st.out == sch.OUT_SEND)
    assert all(not (st.tag & sch.TAG_STRATIFIED) for st in strat if st.out != sch.OUT_SEND)
    world, n = 8, 32 * 1024
    xs = [heavy_tail_grad(n, 30 + r) for r in range(world)]
    exact = np.mean(np.stack(xs).astype(np.float64), 0)
    a = cb.simulate_allreduce(xs, 4, "direct", seed=9)
    b = cb.simulate_allreduce(xs, 4, "direct", seed=9, correlated=True)
    assert all(np.array_equal(b[0], o) for o in b)
    assert cr.nmse(b[0], exact) < cr.nmse(a[0], exact)
