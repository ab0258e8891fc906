"""Checkpoint / resume of model, optimizer, schedule and hook state.

The reference's testbed trainers parse ``--resume_dir`` / ``--last_step`` but never use them
(testbed_evaluation/train_llm_causal.py:204-206); its simulation trainers can only load
(``accelerator.load_state``, simulations_llm/distributed_llm_clm.py:394-415) and never persist the
hook state (controller ``u``, thresholds, random-pool seeds).  Here one file per rank-0 save holds
everything, including the hook's step counter and bit-allocation state; because the stochastic
rounding is a pure function of (seed, step, bucket, position), a resumed run produces the same
codes as an uninterrupted one.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

FORMAT_VERSION = 1


def save(path: str, trainer, extra: Optional[dict] = None) -> None:
    """Write a checkpoint (rank 0 writes; every rank must call, a barrier follows).  The collective engine's
    status is checked first: weights that a timed-out collective left half reduced are never written."""
    if hasattr(trainer, "check"):
        trainer.check()
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        state = {
            "version": FORMAT_VERSION,
            "step": trainer.step_idx,
            "train_config": dict(vars(trainer.cfg)),
            "model": trainer.model.state_dict(),
            "optimizer": trainer.opt.state_dict(),
            "scheduler": trainer.sched.state_dict(),
            "hook": trainer.state.state_dict() if trainer.state is not None else None,
            "extra": extra or {},
        }
        tmp = path + ".tmp"
        torch.save(state, tmp)
        os.replace(tmp, path)
    if dist.is_initialized():
        dist.barrier()


def load(path: str, trainer) -> dict:
    """Restore a trainer in place; returns the ``extra`` dict of the checkpoint."""
    state = torch.load(path, map_location=trainer.device, weights_only=False)
    if state.get("version") != FORMAT_VERSION:
        raise ValueError(f"unsupported checkpoint version {state.get('version')}")
    trainer.model.load_state_dict(state["model"])
    if getattr(trainer, "shadows", None):
        from .ops.linear import enable_shadows

        enable_shadows(trainer.model)  # refresh the bf16 working copies from the restored weights
    trainer.opt.load_state_dict(state["optimizer"])
    trainer.sched.load_state_dict(state["scheduler"])
    trainer.step_idx = int(state["step"])
    if trainer.state is not None and state.get("hook") is not None:
        trainer.state.load_state_dict(state["hook"])
    return state.get("extra", {})
