"""Evaluation-matrix launcher: methods x tasks on one multi-GPU box.

Single-box replacement of the reference's SGE / ssh launch scripts
(testbed_evaluation/submit_qsub_llm_hook_matrix.zsh, qsub_llm_hook_matrix_node.zsh): it expands
the same default matrix (:20-21), applies ``--topology butterfly`` by suffixing the method names
(:232-251), derives a port per combination, runs ``torch.distributed.run`` per combination, keeps
``command.log`` and a ``status`` file per combination and honours ``--continue-on-failure``
(qsub_llm_hook_matrix_node.zsh:412-424).  ``--dry-run`` prints the commands and runs nothing.

Per run directory, as the node script leaves them (:295-333, :403-417): ``metadata.log`` (date, host, package
version, python, torch / CUDA / NCCL versions, visible GPUs, the matrix, ``nvidia-smi -L`` and ``topo -m`` when the
tool is there), per combination ``command.log``, ``launcher.out`` / ``launcher.err``, ``status`` (the launcher's exit
code) and ``rank_<r>.exitcode`` for every rank that ended (written by the trainer, 0 or 1; a rank that was killed
leaves none, which ``status`` then lists as ``missing``), plus ``ranks/`` with one stdout / stderr file per rank
(``torch.distributed.run --log-dir --redirects 3``).

``--nsys-profile-step N`` (qsub_smoke_new_comm_hooks_node.zsh:76-79, :300-312) wraps the launch in
``nsys profile --capture-range=cudaProfilerApi --capture-range-end=stop`` with the trace domains of ``--nsys-trace``
and passes ``--nsys_profile_step N`` to the trainer, which brackets that step with ``cudaProfilerStart / Stop``.  The
wrap is only built when an ``nsys`` binary is found (``--nsys-bin`` or PATH); otherwise the launcher says so and runs
the step markers alone.  ``--numa-node K`` prefixes ``numactl --cpunodebind=K --membind=K`` (:396-398) when numactl
exists.
"""
from __future__ import annotations

import argparse
import datetime
import os
import shlex
import shutil
import socket
import subprocess
import sys
import time
from typing import List, Optional

DEFAULT_METHODS = ("bf16,MXfp8,fp4,fp6,zero,dynamiQ_aee_5bit,dynamiQ_mee_5bit,"
                   "dynamiQ_mee_5bit_dynamic_bitrate,omnireduce,thc")
TASKS = {
    "causal:gpt2-small": ("causal_lm", "gpt2-small", 8, 1024),
    "causal:llama-1.2b": ("causal_lm", "llama-1.2b", 4, 2048),
    "mlm:bert-base": ("masked_lm", "bert-base", 16, 512),
    "mlm:bert-large": ("masked_lm", "bert-large", 8, 512),
    "causal:gpt2-tiny": ("causal_lm", "gpt2-tiny", 2, 32),  # seconds on CPU ranks: the launcher's own test
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
            if args.nsys_profile_step >= 0:
                cmd += ["--nsys_profile_step", str(args.nsys_profile_step)]
            # per-rank stdout / stderr under <out>/ranks (redirect 3 = both streams)
            at = cmd.index("-m", 3)
            cmd[at:at] = ["--log-dir", os.path.join(out, "ranks"), "--redirects", "3"]
            cmd = wrap_profiler(cmd, out, args) if args.nsys_profile_step >= 0 else cmd
            if args.numa_node is not None and shutil.which("numactl"):
                cmd = ["numactl", f"--cpunodebind={args.numa_node}", f"--membind={args.numa_node}"] + cmd
            cmds.append({"task": task, "method": method, "out": out, "cmd": cmd})
    return cmds


def nsys_binary(args) -> Optional[str]:
    return args.nsys_bin if args.nsys_bin and os.path.exists(args.nsys_bin) else shutil.which("nsys")


def wrap_profiler(cmd: List[str], out: str, args) -> List[str]:
    """``nsys profile`` around the whole launch, capturing only between cudaProfilerStart and Stop."""
    nsys = nsys_binary(args)
    if nsys is None:
        return cmd
    return [nsys, "profile", f"--trace={args.nsys_trace}", "--capture-range=cudaProfilerApi",
            "--capture-range-end=stop", "--force-overwrite=true",
            "--output", os.path.join(out, f"nsys_step{args.nsys_profile_step}")] + cmd


def _tool(cmd: List[str]) -> str:
    if shutil.which(cmd[0]) is None:
        return f"({cmd[0]} not found)\n"
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=60).stdout
    except (OSError, subprocess.SubprocessError) as e:
        return f"({' '.join(cmd)} failed: {e})\n"


def write_metadata(path: str, args, cmds: List[dict]) -> None:
    import torch

    from .. import __version__ as version

    lines = [f"date={datetime.datetime.now().astimezone().isoformat(timespec='seconds')}",
             f"host={socket.gethostname()}", f"package_version={version}", f"python={sys.executable}",
             f"torch={torch.__version__}", f"cuda={torch.version.cuda}",
             f"nccl={'.'.join(str(v) for v in torch.cuda.nccl.version()) if torch.cuda.is_available() else 'n/a'}",
             f"gpus={args.gpus}", f"cuda_visible_devices={os.environ.get('CUDA_VISIBLE_DEVICES', '')}",
             f"tasks={args.tasks}", f"methods={','.join(sorted({c['method'] for c in cmds}))}",
             f"topology={args.topology}", f"max_train_steps={args.max_train_steps}",
             f"nsys_profile_step={args.nsys_profile_step}", f"nsys_trace={args.nsys_trace}",
             f"nsys_binary={nsys_binary(args) or 'not found'}", f"numa_node={args.numa_node}"]
    lines += [f"{k}={v}" for k, v in sorted(os.environ.items()) if k.startswith(("DQ_", "NCCL_"))]
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
        f.write(_tool(["nvidia-smi", "-L"]))
        f.write(_tool(["nvidia-smi", "topo", "-m"]))


def rank_exit_codes(out: str, world: int) -> List[str]:
    codes = []
    for r in range(world):
        try:
            with open(os.path.join(out, f"rank_{r}.exitcode")) as f:
                codes.append(f.read().strip())
        except OSError:
            codes.append("missing")
    return codes


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
    ap.add_argument("--nsys-profile-step", "--nsys_profile_step", type=int, default=-1,
                    help="capture this training step under nsys (cudaProfilerApi capture range)")
    ap.add_argument("--nsys-trace", "--nsys_trace", default="cuda,nvtx,osrt")
    ap.add_argument("--nsys-bin", default="/usr/local/cuda/bin/nsys")
    ap.add_argument("--numa-node", "--numa_node", type=int, default=None)
    args = ap.parse_args(argv)
    cmds = build_commands(args)
    failures = 0
    if not args.dry_run:
        os.makedirs(args.output_root, exist_ok=True)
        write_metadata(os.path.join(args.output_root, "metadata.log"), args, cmds)
        if args.nsys_profile_step >= 0 and nsys_binary(args) is None:
            print("[run_matrix] no nsys binary found: the step is marked with cudaProfilerStart / Stop and NVTX "
                  "ranges, but nothing records them", flush=True)
    for c in cmds:
        line = " ".join(shlex.quote(x) for x in c["cmd"])
        if args.dry_run:
            print(line)
            continue
        os.makedirs(c["out"], exist_ok=True)
        stamp = datetime.datetime.now().astimezone().isoformat(timespec="seconds")
        with open(os.path.join(c["out"], "command.log"), "w") as f:
            f.write(f"date={stamp}\ntask={c['task']}\naggregation_method={c['method']}\ncommand={line}\n")
        print(f"[{stamp}] task={c['task']} method={c['method']} start", flush=True)
        with open(os.path.join(c["out"], "launcher.out"), "w") as so, open(os.path.join(c["out"], "launcher.err"), "w") as se:
            rc = subprocess.call(c["cmd"], stdout=so, stderr=se)
        codes = rank_exit_codes(c["out"], args.gpus)
        with open(os.path.join(c["out"], "status"), "w") as f:
            f.write(f"exitcode {rc}\n" + "".join(f"rank {r} {code}\n" for r, code in enumerate(codes)))
        print(f"[{datetime.datetime.now().astimezone().isoformat(timespec='seconds')}] task={c['task']} "
              f"method={c['method']} exit={rc} ranks={','.join(codes)}", flush=True)
        if rc != 0:
            failures += 1
            if not args.continue_on_failure:
                return rc
    return 1 if failures else 0


if __name__ == "__main__":
    raise SystemExit(main())
