"""Momentum thresholds, command-file poller, THC constants."""
import os

import torch

from dynamiq_sigcomm_artifact_b200 import bitalloc
from dynamiq_sigcomm_artifact_b200.config import parse_method
from dynamiq_sigcomm_artifact_b200.launch.poller import CommandFilePoller
from dynamiq_sigcomm_artifact_b200.parallel import thc_tables


def test_momentum_thresholds_track_quantiles():
    spec = parse_method("dynamiQ_mee_5bit_momentum")
    assert spec.family == "superchunk" and spec.momentum and not spec.dynamic_bitrate
    thr = {8: 0.2, 4: 0.6, 2: 0.2}
    m = bitalloc.MomentumThresholds(thr)
    g = torch.Generator().manual_seed(0)
    frac = None
    for _ in range(40):
        e1, e2 = torch.exp(torch.randn(3000, generator=g) * 2 - 9), torch.exp(torch.randn(1000, generator=g) * 2 - 9)
        w = torch.cat([m.widths(e1), m.widths(e2)])
        assert set(w.tolist()) <= {2, 4, 8}
        frac = [(w == b).float().mean().item() for b in (8, 4, 2)]
        m.end_of_step()
    assert abs(frac[0] - 0.2) < 0.05 and abs(frac[1] - 0.6) < 0.06 and abs(frac[2] - 0.2) < 0.05, frac
    sd = m.state_dict()
    m2 = bitalloc.MomentumThresholds(thr)
    m2.load_state_dict(sd)
    assert torch.equal(m2.state, m.state)
    gr = m2.groups(torch.tensor([1.0, 1e-9, sd["kth"] * 0.5]))
    assert gr[8].tolist() == [0] and gr[2].tolist() == [1] and gr[4].tolist() == [2]


def test_command_file_poller_runs_new_lines_once(tmp_path):
    path = tmp_path / "commands.txt"
    path.write_text("echo one\ncd sub\n\necho two\nhalf written")
    ran = []
    p = CommandFilePoller(str(path), global_seed=7, poll_seconds=0.0,
                          runner=lambda cmd, env, cwd: ran.append((cmd, env["GLOBAL_SEED"], os.path.basename(cwd))) or 0)
    assert p.poll_once() and [r[0] for r in ran] == ["echo one", "echo two"]
    assert ran[0][1] == "7" and ran[1][2] == "sub"
    assert p.poll_once() and len(ran) == 2  # nothing new: the unfinished line waits for its newline
    with open(path, "a") as f:
        f.write("\nexit\necho never\n")
    assert not p.poll_once()
    assert [r[0] for r in ran] == ["echo one", "echo two", "half written"]
    assert p.run(max_polls=1) == 3


def test_thc_threshold_is_the_two_sided_normal_quantile():
    assert abs(thc_tables.clip_threshold(2.0 ** -10) - thc_tables.THC_T) < 1e-9
    assert abs(thc_tables.clipping_error(0.0) - 1.0) < 1e-9  # everything clipped to zero: E[x^2]
    e31, e255 = thc_tables.expected_error(thc_tables.THC_T, 31), thc_tables.expected_error(thc_tables.THC_T, 255)
    assert 0.0 < e255 < e31 < 0.02
    t_best, e_best = thc_tables.best_threshold(31)
    assert 2.0 < t_best < thc_tables.THC_T and e_best <= e31


def test_threshold_widths_agree_with_group_split():
    from dynamiq_sigcomm_artifact_b200.config import THRESHOLD_TABLE

    g = torch.Generator().manual_seed(5)
    for key in ("3bit", "5bit", "7bit", "4bit_fixed"):
        thr = THRESHOLD_TABLE[key]
        e = torch.exp(torch.randn(1003, generator=g) * 3)
        e[10:20] = e[10]  # ties keep their original order (stable sort)
        widths = bitalloc.threshold_widths(e, thr)
        groups = bitalloc.split_by_thresholds(e, thr)
        for b in (8, 4, 2):
            assert sorted(torch.nonzero(widths == b).reshape(-1).tolist()) == sorted(groups[b].tolist()), (key, b)
        assert widths.dtype == torch.uint8 and int((widths == 0).sum()) == 0


def test_flat_bucket_quacks_like_a_grad_bucket():
    from dynamiq_sigcomm_artifact_b200.parallel.reducer import FlatBucket

    p = torch.nn.Parameter(torch.zeros(6))
    buf = torch.arange(6.0)
    p.grad = buf.view_as(p)
    b = FlatBucket(3, buf, [p], last=True)
    assert b.index() == 3 and b.is_last() and b.buffer() is buf
    assert b.parameters() == [p] and b.gradients()[0].data_ptr() == buf.data_ptr()
    b.set_buffer(torch.ones(6))
    assert torch.equal(buf, torch.ones(6))
    b.set_buffer(buf)  # the same storage: nothing to copy
    assert torch.equal(p.grad, torch.ones(6))


def test_level_solver_reproduces_the_published_optima():
    """Errors and positions of the reference's result files (simulations_llm/compression/
    optimal_INCA_2_X_bits_invp_1024.txt and optimal_INCA_5_X_bits_invp_1024_n16.txt), read as text."""
    golden2 = {3: (0.8130913915224226, [1, 3]), 4: (0.6293661377218382, [1, 4]), 9: (0.6267778470922883, [2, 9])}
    for g, (err, pos) in golden2.items():
        e, p = thc_tables.solve_levels(2, g)
        assert abs(e - err) < 1e-12 and p == pos, (g, e, p)
    e, p = thc_tables.solve_levels(5, 16)
    assert abs(e - 0.0071314959952194935) < 1e-12 and p == list(range(15)) + [16]
    e, p = thc_tables.solve_levels(5, 2)
    assert abs(e - 0.45248911821625015) < 1e-12 and p[-2:] == [1, 2] and set(p[:-2]) == {0}
    assert abs(thc_tables.solve_levels(2, 1)[0] - 1.6317562270095627) < 1e-12
    # a finer grid never hurts, and the optimum beats the uniform grid of the same size
    errs = [thc_tables.solve_levels(4, g)[0] for g in (8, 12, 21, 40)]
    assert all(a >= b - 1e-15 for a, b in zip(errs, errs[1:]))
    uniform = sum(thc_tables.interval_cost(-thc_tables.THC_T + i * 2 * thc_tables.THC_T / 15,
                                           -thc_tables.THC_T + (i + 1) * 2 * thc_tables.THC_T / 15) for i in range(15))
    assert errs[-1] < uniform


def test_sender_and_receiver_tables_are_unbiased_and_summable():
    g, bits = 21, 4
    _, pos = thc_tables.solve_levels(bits, g)
    recv = thc_tables.receiver_table(pos, g)
    levels = thc_tables.level_values(pos, g)
    assert recv[0] == 0 and recv[-1] == 2 * g and recv == sorted(recv) and len(recv) == 1 << bits
    lower, prob = thc_tables.sender_table(pos, g, 1001)
    T = thc_tables.THC_T
    for q in (0, 137, 500, 730, 1000):  # E[decoded] equals the fine-grid input
        x = -T + 2 * T * q / 1000
        k, p = lower[q], prob[q]
        assert abs((1 - p) * levels[k] + p * levels[k + 1] - x) < 1e-12
    # integer sums decode linearly: two senders' table values
    a, b = recv[3], recv[12]
    assert abs(((a + b) - 2 * g) * T / g - (levels[3] + levels[12])) < 1e-12
