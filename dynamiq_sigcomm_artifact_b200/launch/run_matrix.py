"""Evaluation-matrix launcher: methods x tasks on one multi-GPU box.

Single-box replacement of the reference's SGE / ssh launch scripts
(testbed_evaluation/submit_qsub_llm_hook_matrix.zsh, qsub_llm_hook_matrix_node.zsh): it expands
the same default matrix (:20-21), applies ``--topology butterfly`` by suffixing the method names
(:232-251), derives a port per combination, runs ``torch.distributed.run`` per combination, keeps
``command.log`` and a ``status`` file per combination and honours ``--continue-on-failure``
(qsub_llm_hook_matrix_node.zsh:412-424).  ``--dry-run`` prints the commands and runs nothing.
"""
from __future__ import annotations

import argparse
import os
import shlex
import subprocess
import sys
import time
from typing import List

DEFAULT_METHODS = ("bf16,MXfp8,fp4,fp6,zero,dynamiQ_aee_5bit,dynamiQ_mee_5bit,"
                   "dynamiQ_mee_5bit_dynamic_bitrate,omnireduce,thc")
TASKS = {
    "causal:gpt2-small": ("causal_lm", "gpt2-small", 8, 1024),
    "causal:llama-1.2b": ("causal_lm", "llama-1.2b", 4, 2048),
    "mlm:bert-base": ("masked_lm", "bert-base", 16, 512),
    "mlm:bert-large": ("masked_lm", "bert-large", 8, 512),
}


def normalise_methods(methods: List[str], topology: str) -> List[str]:
    out = []
    for m in methods:
        if topology in ("butterfly", "direct") and topology not in m.lower() and m.lower() not in ("zero",):
            m = f"{m}_{topology}"
        out.append(m)
    return out


def build_commands(args) -> List[dict]:
    methods = normalise_methods([m for m in args.aggregation_methods.split(",") if m], args.topology)
    tasks = [t for t in args.tasks.split(",") if t]
    base_port = args.base_port or 20000 + int(time.time()) % 20000
    cmds = []
    for ti, task in enumerate(tasks):
        module, model, batch, seq = TASKS[task]
        for mi, method in enumerate(methods):
            out = os.path.join(args.output_root, task.replace(":", "_"), method)
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(base_port + ti * 100 + mi),
                   "-m", f"dynamiq_sigcomm_artifact_b200.train.{module}", "--model_name", model,
                   "--aggregation_method", method, "--per_device_train_batch_size", str(batch),
                   "--block_size", str(seq), "--max_train_steps", str(args.max_train_steps),
                   "--output_dir", out]
            if args.measure_comm_error:
                cmd.append("--measure_comm_error")
            cmds.append({"task": task, "method": method, "out": out, "cmd": cmd})
    return cmds


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--aggregation-methods", "--aggregation_methods", default=DEFAULT_METHODS)
    ap.add_argument("--tasks", default="causal:llama-1.2b,causal:gpt2-small,mlm:bert-base")
    ap.add_argument("--topology", default="direct", choices=["ring", "butterfly", "direct"])
    ap.add_argument("--max-train-steps", "--max_train_steps", type=int, default=151)
    ap.add_argument("--output-root", "--output_root", default="matrix_results")
    ap.add_argument("--base-port", type=int, default=0)
    ap.add_argument("--measure-comm-error", action="store_true")
    ap.add_argument("--continue-on-failure", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    cmds = build_commands(args)
    failures = 0
    for c in cmds:
        line = " ".join(shlex.quote(x) for x in c["cmd"])
        if args.dry_run:
            print(line)
            continue
        os.makedirs(c["out"], exist_ok=True)
        with open(os.path.join(c["out"], "command.log"), "w") as f:
            f.write(line + "\n")
        rc = subprocess.call(c["cmd"])
        with open(os.path.join(c["out"], "status"), "w") as f:
            f.write(f"exitcode {rc}\n")
        if rc != 0:
            failures += 1
            if not args.continue_on_failure:
                return rc
    return 1 if failures else 0


if __name__ == "__main__":
    raise SystemExit(main())
