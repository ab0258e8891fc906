"""Shared driver of the training entry points (causal LM and masked LM).

Follows the reference's measurement protocol: optimizer steps ``MEASURE_START_STEP`` (4) to
``MEASURE_END_STEP`` (150) are timed with a device synchronisation at both ends and rank 0 writes
``measured_steps N elapsed_seconds X avg_seconds_per_step Y`` to ``results.txt``
(testbed_evaluation/train_llm_causal.py:46-47,359-393); interim progress every 10 steps (:363-365);
``config.txt`` / ``log.txt`` in the output directory (:634-641).  Data are synthetic token ids of
the requested shape (there are no datasets here); the MLM task masks 15 % of the positions
80/10/10 as the reference does (train_llm_maskedlm_bert.py:354-385).
"""
from __future__ import annotations

import argparse
import os
import time

import torch
import torch.distributed as dist

from .. import checkpoint
from ..utils import tracing
from ..utils.metrics import RunLog
from .engine import TrainConfig, Trainer

MEASURE_START_STEP = 4
MEASURE_END_STEP = 150


def default_lr(task: str, world: int, model: str = "") -> float:
    """The launch scripts' rule base * sqrt(W / 2) * (8 / W) ** 0.4
    (testbed_evaluation/qsub_llm_hook_matrix_node.zsh:196-215); MLM uses a constant 5e-5."""
    if task == "mlm":
        return 5e-5
    base = 1e-5 * (0.7 if "gemma" in model else 1.0)
    w = max(world, 1)
    return base * (w / 2) ** 0.5 * (8 / w) ** 0.4


def evaluate(tr: Trainer, batches: int):
    """Mean loss and perplexity over held-out synthetic batches, averaged over ranks
    (simulations_llm/distributed_llm_clm.py:350-374)."""
    import math

    tr.model.eval()
    total = 0.0
    saved = tr.step_idx
    with torch.no_grad():
        for i in range(batches):
            tr.step_idx = 10_000_000 + i  # batches the training loop never sees
            ids = tr.synthetic_batch(pinned=False).to(tr.device)
            if tr.cfg.task == "mlm":
                from ..models import mask_tokens

                c = tr.model.config
                x, y = mask_tokens(ids, c.vocab, c.mask_token_id, tr._gen)
                total += float(tr.model(x, y))
            else:
                total += float(tr.model(ids, ids))
    tr.step_idx = saved
    tr.model.train()
    mean = torch.tensor([total / max(batches, 1)], dtype=torch.float64, device=tr.device)
    if dist.is_initialized():
        dist.all_reduce(mean)
        mean /= dist.get_world_size()
    m = float(mean)
    return m, math.exp(min(m, 50.0))


def build_parser(task: str, default_model: str, default_seq: int, default_batch: int) -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=f"{task} training throughput / accuracy run on synthetic tokens")
    ap.add_argument("--model_name", "--model", default=default_model)
    ap.add_argument("--aggregation_method", "--aggregation-method", default="dynamiQ_aee_5bit")
    ap.add_argument("--topology", default=None, choices=[None, "ring", "butterfly", "direct"])
    ap.add_argument("--per_device_train_batch_size", type=int, default=default_batch)
    ap.add_argument("--block_size", type=int, default=default_seq)
    ap.add_argument("--learning_rate", type=float, default=None)
    ap.add_argument("--weight_decay", type=float, default=0.0)
    ap.add_argument("--max_train_steps", type=int, default=MEASURE_END_STEP + 1)
    ap.add_argument("--measure_start_step", type=int, default=MEASURE_START_STEP)
    ap.add_argument("--measure_end_step", type=int, default=MEASURE_END_STEP)
    ap.add_argument("--bucket_cap_mb", type=int, default=0, help="0: one bucket for the package's own collectives, 25 MB for the library all-reduce")
    ap.add_argument("--comm_ctas", type=int, default=64)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--output_dir", default=None)
    ap.add_argument("--resume_from", default=None, help="checkpoint file written by --checkpointing_steps")
    ap.add_argument("--checkpointing_steps", type=int, default=0)
    ap.add_argument("--measure_comm_error", action="store_true")
    ap.add_argument("--enable_nvtx", action="store_true")
    ap.add_argument("--nsys_profile_step", type=int, default=-1)
    ap.add_argument("--eval_batches", type=int, default=0, help="held-out batches for a final loss / perplexity")
    ap.add_argument("--gradient_accumulation_steps", type=int, default=1,
                    help="accepted for command-line compatibility; the reference parses it and never uses it")
    return ap


def main(task: str, argv=None, default_model: str = "gpt2-small", default_seq: int = 1024, default_batch: int = 8):
    """Parse, train, and leave ``rank_<r>.exitcode`` (0, or 1 after an exception, which is re-raised) in the
    output directory: the launcher collects one per rank, since the process launcher reports a single code."""
    args = build_parser(task, default_model, default_seq, default_batch).parse_args(argv)
    code = 1
    try:
        loss = _run(task, args)
        code = 0
        return loss
    finally:
        if args.output_dir:
            os.makedirs(args.output_dir, exist_ok=True)
            with open(os.path.join(args.output_dir, f"rank_{os.environ.get('RANK', '0')}.exitcode"), "w") as f:
                f.write(f"{code}\n")


def _run(task: str, args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    use_cuda = torch.cuda.is_available()
    if world > 1:
        if use_cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl" if use_cuda else "gloo")
    rank = dist.get_rank() if dist.is_initialized() else 0
    tracing.enable(args.enable_nvtx)
    lr = args.learning_rate if args.learning_rate is not None else default_lr(task, world, args.model_name)
    cfg = TrainConfig(model=args.model_name, method=args.aggregation_method, micro_batch=args.per_device_train_batch_size,
                      seq_len=args.block_size, lr=lr, weight_decay=args.weight_decay, total_steps=args.max_train_steps,
                      bucket_cap_mb=args.bucket_cap_mb, seed=args.seed, task=task, topology=args.topology,
                      comm_ctas=args.comm_ctas, measure_comm_error=args.measure_comm_error,
                      dtype="bf16" if use_cuda else "fp32")
    log = RunLog(args.output_dir, rank)
    log.config({**vars(args), "world_size": world, "learning_rate_used": lr})
    tr = Trainer(cfg)
    if args.resume_from:
        checkpoint.load(args.resume_from, tr)
        log.log(f"resumed from {args.resume_from} at step {tr.step_idx}")
    window = tracing.ProfilerWindow(args.nsys_profile_step)
    t_start, measured = None, 0
    loss = float("nan")
    while tr.step_idx < args.max_train_steps:
        step = tr.step_idx
        if step == args.measure_start_step:
            if use_cuda:
                torch.cuda.synchronize()
            t_start = time.perf_counter()
        window.before(step)
        with tracing.nvtx_range(f"rank{rank}.step{step}"):
            loss = tr.train_step(tr.synthetic_batch())
        window.after(step)
        if t_start is not None and step < args.measure_end_step:
            measured += 1
        if step % 10 == 0 and rank == 0:
            el = f" elapsed={time.perf_counter() - t_start:.3f}" if t_start is not None else ""
            log.log(f"batch_idx={step} loss={loss:.4f}{el}")
        if args.measure_comm_error and tr.state is not None:
            st = tr.state["stats"]
            log.vnmse(step, st["err_sq"], st["ref_sq"])
        if args.checkpointing_steps and (step + 1) % args.checkpointing_steps == 0 and args.output_dir:
            checkpoint.save(os.path.join(args.output_dir, f"step_{step + 1}.pt"), tr)
        if t_start is not None and step + 1 == min(args.measure_end_step, args.max_train_steps):
            if use_cuda:
                torch.cuda.synchronize()
            elapsed = time.perf_counter() - t_start
            tr.check()  # no results line from a run whose collectives gave up on a wait
            line = log.results(measured, elapsed)
            if rank == 0:
                print(line, flush=True)
    if args.eval_batches > 0:
        ppl = evaluate(tr, args.eval_batches)
        log.log(f"eval_loss={ppl[0]:.4f} perplexity={ppl[1]:.2f}")
    tr.check()
    tr.close()
    if dist.is_initialized():
        dist.destroy_process_group()
    return loss
