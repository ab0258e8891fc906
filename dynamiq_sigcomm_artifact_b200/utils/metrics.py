"""Result files and bandwidth definitions, in the reference's formats.

* ``results.txt``: ``measured_steps N elapsed_seconds X avg_seconds_per_step Y``
  (testbed_evaluation/train_llm_causal.py:386-393);
* ``comm_error_vnmse.tsv``: accumulated ``||ret - gt||^2`` and ``||gt||^2`` per step
  (simulations_llm/new_comm_hooks/comm_hooks.py:22-50,1167-1198);
* ``algbw`` and wire bandwidth as in rdma_comm_compress/sample_allreduce.py:721-727.
"""
from __future__ import annotations

import json
import os
import time
from typing import Optional


def algbw_gbs(input_bytes: int, world: int, seconds: float) -> float:
    """2 (W-1) / W x input bytes / t, in GB/s."""
    return 2 * (world - 1) / world * input_bytes / seconds / 1e9


def wire_gbs(message_bytes: int, world: int, seconds: float) -> float:
    """Bytes that cross a rank's link in one direction: 2 (W-1) messages of one shard."""
    return 2 * (world - 1) * message_bytes / seconds / 1e9


class RunLog:
    """log.txt / config.txt / results.txt in an output directory (rank 0 only)."""

    def __init__(self, out_dir: Optional[str], rank: int = 0):
        self.dir = out_dir if (out_dir and rank == 0) else None
        if self.dir:
            os.makedirs(self.dir, exist_ok=True)

    def config(self, cfg: dict) -> None:
        if self.dir:
            with open(os.path.join(self.dir, "config.txt"), "w") as f:
                json.dump(cfg, f, indent=1, default=str)

    def log(self, msg: str) -> None:
        line = f"[{time.strftime('%H:%M:%S')}] {msg}"
        print(line, flush=True)
        if self.dir:
            with open(os.path.join(self.dir, "log.txt"), "a") as f:
                f.write(line + "\n")

    def results(self, measured_steps: int, elapsed_seconds: float) -> str:
        line = (f"measured_steps {measured_steps} elapsed_seconds {elapsed_seconds:.6f} "
                f"avg_seconds_per_step {elapsed_seconds / max(measured_steps, 1):.6f}")
        if self.dir:
            with open(os.path.join(self.dir, "results.txt"), "w") as f:
                f.write(line + "\n")
        return line

    def vnmse(self, step: int, err_sq: float, ref_sq: float) -> None:
        if not self.dir:
            return
        path = os.path.join(self.dir, "comm_error_vnmse.tsv")
        new = not os.path.exists(path)
        with open(path, "a") as f:
            if new:
                f.write("step\terr_sq\tref_sq\tvnmse\n")
            f.write(f"{step}\t{err_sq:.9e}\t{ref_sq:.9e}\t{(err_sq / ref_sq if ref_sq > 0 else 0.0):.9e}\n")
