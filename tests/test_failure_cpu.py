"""Failure detection without a GPU fault: lost messages, a rank that never joins, bad handshakes."""
import os
import socket
from datetime import timedelta

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dynamiq_sigcomm_artifact_b200.parallel import cpu_backend as cb
from dynamiq_sigcomm_artifact_b200.parallel.fused import CollectiveTimeout, decode_status
from dynamiq_sigcomm_artifact_b200.parallel.symm import RankMeta, TopologyError, validate_metas

from helpers import heavy_tail_grad


def test_lost_message_ends_in_a_timeout_not_a_hang():
    xs = [heavy_tail_grad(4096, r) for r in range(4)]
    lossy = cb.LocalTransport(4, timeout=0.5, drop=lambda src, dst, slot: (src, dst, slot) == (1, 2, 1))
    with pytest.raises(TimeoutError, match="slot"):
        cb.simulate_allreduce(xs, 4, "ring", transport=lossy)
    ok = cb.simulate_allreduce(xs, 4, "ring", transport=cb.LocalTransport(4, timeout=5.0))
    assert all(np.array_equal(ok[0], o) for o in ok)


def test_status_word_decoding():
    assert decode_status([0, 0, 0, 0]) is None
    msg = decode_status([1, (5 << 16) | 17, 3, 0])
    assert "timed out" in msg and "step 5" in msg and "CTA 17" in msg and "slot 3" in msg
    assert "bulk copy" in decode_status([3, 0, 0, 0])
    assert issubclass(CollectiveTimeout, RuntimeError)


def _meta(rank, host="box", device=None, handle=b"x" * 64):
    return RankMeta(rank, host, rank if device is None else device, "NVIDIA B200", handle)


def test_handshake_validation_rejects_bad_layouts():
    p2p = [[[1, 0, 1] for _ in range(4)] for _ in range(4)]
    validate_metas([_meta(r) for r in range(4)], 0, p2p)
    with pytest.raises(TopologyError, match="one host"):
        validate_metas([_meta(0), _meta(1, host="other")], 0, p2p)
    with pytest.raises(TopologyError, match="share a GPU"):
        validate_metas([_meta(0), _meta(1, device=0)], 0, p2p)
    with pytest.raises(TopologyError, match="out of order"):
        validate_metas([_meta(1), _meta(0)], 0, p2p)
    with pytest.raises(TopologyError, match="IPC handle"):
        validate_metas([_meta(0), _meta(1, handle=b"short")], 0, p2p)
    with pytest.raises(TopologyError, match="did not publish"):
        validate_metas([_meta(0), None], 0, p2p)
    p2p[0][1][0] = 0
    with pytest.raises(TopologyError, match="peer-to-peer"):
        validate_metas([_meta(0), _meta(1)], 0, p2p)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_that_leaves(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=4))
    x = heavy_tail_grad(8192, rank)
    out = cb.allreduce_gloo(x, 5, "ring", seed=1, step=0, bucket=0)  # one healthy collective first
    if rank == 1:
        q.put(("left", rank))
        os._exit(0)  # leaves between steps, with nothing in flight
    try:
        cb.allreduce_gloo(x, 5, "ring", seed=1, step=1, bucket=0)
        q.put(("no error", rank))
    except Exception as e:  # the short process-group timeout ends the collective with an error
        q.put(("error", type(e).__name__))
    os._exit(0)


def test_rank_that_leaves_between_steps_is_detected_by_timeout():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_that_leaves, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive(), "a rank hung instead of failing"
    got = dict([q.get(), q.get()])
    assert "left" in got and "error" in got, got
