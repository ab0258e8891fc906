"""Entry points, launcher, checkpoint/resume and result files on CPU."""
import os

import numpy as np
import torch

from dynamiq_sigcomm_artifact_b200 import checkpoint
from dynamiq_sigcomm_artifact_b200.launch import run_matrix
from dynamiq_sigcomm_artifact_b200.train import run as train_run
from dynamiq_sigcomm_artifact_b200.train.engine import TrainConfig, Trainer
from dynamiq_sigcomm_artifact_b200.utils import clocks, metrics


def test_launcher_dry_run_expands_matrix(capsys):
    rc = run_matrix.main(["--dry-run", "--gpus", "4", "--topology", "butterfly", "--tasks", "causal:gpt2-small",
                          "--aggregation-methods", "bf16,dynamiQ_aee_5bit,zero", "--base-port", "23000"])
    out = capsys.readouterr().out.strip().splitlines()
    assert rc == 0 and len(out) == 3
    assert "--nproc-per-node=4" in out[0] and "bf16_butterfly" in out[0] and "--master-port 23000" in out[0]
    assert "dynamiQ_aee_5bit_butterfly" in out[1] and "--aggregation_method zero " in out[2] and "zero_butterfly" not in out[2]
    assert run_matrix.DEFAULT_METHODS.split(",")[5] == "dynamiQ_aee_5bit"


def test_launcher_runs_a_combination_and_leaves_its_logs(tmp_path):
    """Two gloo ranks, three steps of the tiny model, under a stand-in for the system profiler that records
    its arguments and runs the command it was given."""
    fake = tmp_path / "nsys"
    fake.write_text("#!/bin/bash\necho \"$@\" > %s\nwhile [ \"$1\" != \"%s\" ]; do shift; done\nexec \"$@\"\n"
                    % (tmp_path / "nsys_args.txt", os.sys.executable))
    fake.chmod(0o755)
    root = tmp_path / "matrix"
    env_before = os.environ.get("CUDA_VISIBLE_DEVICES")
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    try:
        rc = run_matrix.main(["--gpus", "2", "--tasks", "causal:gpt2-tiny", "--aggregation-methods", "dynamiQ_aee_5bit",
                              "--max-train-steps", "3", "--output-root", str(root), "--nsys-profile-step", "1",
                              "--nsys-bin", str(fake), "--base-port", "23450"])
    finally:
        if env_before is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES")
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = env_before
    out = root / "causal_gpt2-tiny" / "dynamiQ_aee_5bit_direct"
    assert rc == 0, (out / "launcher.err").read_text()[-2000:]
    meta = (root / "metadata.log").read_text()
    assert "host=" in meta and "torch=" in meta and "methods=dynamiQ_aee_5bit_direct" in meta and f"nsys_binary={fake}" in meta
    assert (out / "status").read_text().splitlines() == ["exitcode 0", "rank 0 0", "rank 1 0"]
    assert "aggregation_method=dynamiQ_aee_5bit_direct" in (out / "command.log").read_text()
    nsys_args = (tmp_path / "nsys_args.txt").read_text()
    assert "--capture-range=cudaProfilerApi" in nsys_args and "--capture-range-end=stop" in nsys_args
    assert "--trace=cuda,nvtx,osrt" in nsys_args and "--nsys_profile_step 1" in nsys_args
    assert (out / "ranks").is_dir() and any((out / "ranks").rglob("stdout.log"))


def test_lr_rule_and_bandwidth_definitions():
    assert abs(train_run.default_lr("causal", 8) - 1e-5 * 2.0) < 1e-12
    assert abs(train_run.default_lr("causal", 2) - 1e-5 * (4 ** 0.4)) < 1e-12
    assert train_run.default_lr("mlm", 8) == 5e-5
    assert abs(metrics.algbw_gbs(1 << 30, 8, 1.0) - 2 * 7 / 8 * (1 << 30) / 1e9) < 1e-9
    assert abs(metrics.wire_gbs(146, 8, 1.0) - 14 * 146 / 1e9) < 1e-15


def test_clock_summary_parses_nvidia_smi_lines():
    lines = ["0, 1365, 1965, 950.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
             "0, 1410, 1965, 990.0, 0x0, Not Active, Not Active, Not Active, Not Active", "garbage"]
    s = clocks.summarise(lines)
    assert s["sm_mhz"] == 1387.5 and s["sm_max_mhz"] == 1965.0 and s["reasons"] == ["sw_power_cap"] and s["samples"] == 2


def test_entry_point_writes_results_and_resumes(tmp_path):
    out = str(tmp_path / "run")
    argv = ["--model_name", "gpt2-tiny", "--per_device_train_batch_size", "2", "--block_size", "32",
            "--max_train_steps", "8", "--measure_start_step", "2", "--measure_end_step", "8", "--output_dir", out,
            "--checkpointing_steps", "4", "--learning_rate", "1e-3"]
    from dynamiq_sigcomm_artifact_b200.train import causal_lm

    loss_full = causal_lm.main(argv)
    text = open(os.path.join(out, "results.txt")).read().split()
    assert text[0] == "measured_steps" and int(text[1]) == 6 and text[4] == "avg_seconds_per_step"
    assert os.path.exists(os.path.join(out, "step_4.pt")) and os.path.exists(os.path.join(out, "config.txt"))
    loss_resumed = causal_lm.main(argv + ["--resume_from", os.path.join(out, "step_4.pt")])
    assert abs(loss_full - loss_resumed) < 1e-6, "resume does not reproduce the uninterrupted run"


def test_checkpoint_roundtrip_restores_optimizer_state(tmp_path):
    a = Trainer(TrainConfig(model="llama-tiny", micro_batch=2, seq_len=32, lr=1e-3, dtype="fp32"),
                device=torch.device("cpu"))
    for _ in range(3):
        a.train_step(a.synthetic_batch(pinned=False))
    path = str(tmp_path / "ck.pt")
    checkpoint.save(path, a, extra={"note": "x"})
    b = Trainer(TrainConfig(model="llama-tiny", micro_batch=2, seq_len=32, lr=1e-3, dtype="fp32", seed=99),
                device=torch.device("cpu"))
    assert checkpoint.load(path, b) == {"note": "x"} and b.step_idx == 3
    b.cfg.seed = a.cfg.seed
    la = a.train_step(a.synthetic_batch(pinned=False))
    lb = b.train_step(b.synthetic_batch(pinned=False))
    assert abs(la - lb) < 1e-6


def test_masked_lm_masking_statistics():
    from dynamiq_sigcomm_artifact_b200.models import mask_tokens

    g = torch.Generator().manual_seed(0)
    ids = torch.randint(5, 1000, (64, 512), generator=g)
    x, y = mask_tokens(ids, 1000, 3, g)
    sel = y != -100
    frac = float(sel.float().mean())
    assert abs(frac - 0.15) < 0.01
    masked = float((x[sel] == 3).float().mean())
    assert abs(masked - 0.8) < 0.03
    assert bool((x[~sel] == ids[~sel]).all()) and bool((y[sel] == ids[sel]).all())


def test_mmlu_entry_point_learns_the_synthetic_task(tmp_path):
    from dynamiq_sigcomm_artifact_b200.train import mmlu
    from dynamiq_sigcomm_artifact_b200.utils import data

    acc = mmlu.main(["--model_name", "llama-tiny", "--per_device_train_batch_size", "16", "--block_size", "8",
                     "--max_train_steps", "150", "--learning_rate", "3e-3", "--eval_items", "128",
                     "--output_dir", str(tmp_path / "m")])
    assert acc > 0.5  # chance is 0.25
    assert data.format_mmlu_prompt("Q?", ["w", "x", "y", "z"], 2).endswith("Answer: C")
    orders = data.gen_orders(10, 2, 1)
    assert sorted(orders[0]) == list(range(10)) and orders[0] != orders[1]
    assert list(data.PrecomputedSampler(orders[0], 1, 2)) == orders[0][1::2]


def test_eval_reports_perplexity(tmp_path, capsys):
    from dynamiq_sigcomm_artifact_b200.train import masked_lm

    masked_lm.main(["--model_name", "bert-tiny", "--per_device_train_batch_size", "2", "--block_size", "32",
                    "--max_train_steps", "3", "--eval_batches", "2", "--output_dir", str(tmp_path / "b")])
    assert "perplexity=" in capsys.readouterr().out


def test_bucket_policy_and_wire_accounting():
    from dynamiq_sigcomm_artifact_b200.parallel.fused import wire_bytes_per_rank
    from dynamiq_sigcomm_artifact_b200.train.engine import default_bucket_cap_mb

    # one bucket per model for the package's own collectives on several GPUs, small buckets otherwise
    assert default_bucket_cap_mb("dynamiQ_aee_5bit", 8, "gpt2-small") == 4000
    assert default_bucket_cap_mb("bf16", 4, "bert-base") == 4000
    assert default_bucket_cap_mb("fp32", 8, "gpt2-small") == 25 and default_bucket_cap_mb("none", 2, "x") == 25
    assert default_bucket_cap_mb("dynamiQ_aee_5bit", 1, "gpt2-small") == 25
    assert default_bucket_cap_mb("dynamiQ_aee_5bit", 1, "llama-1.2b") == 100
    # bytes per rank and direction: 2 (W - 1) shards; rotation codec 128 b + 4 per block, bf16 wire 2 KiB per block
    n, w = 8 * 1024 * 16, 4
    assert wire_bytes_per_rank(n, w, 5, "rht") == 2 * 3 * 32 * 644
    assert wire_bytes_per_rank(n, w, 4.5, "rht_mix") == 2 * 3 * 32 * 580
    assert wire_bytes_per_rank(n, w, 16, "cast") == 2 * 3 * 32 * 2048
    assert wire_bytes_per_rank(n, w, 4, "scmix_mee") == 2 * 3 * 32 * 4 * 146
    assert wire_bytes_per_rank(n, 1, 5, "rht") == 0
