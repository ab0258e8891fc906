"""MMLU-style fine-tuning entry point: causal LM, loss at the answer position, letter accuracy.

Counterpart of testbed_evaluation/train_llm_mmlu.py (throughput) and
simulations_llm/distributed_llm_mmlu.py (accuracy), on a synthetic multiple-choice set.  As the
reference does (train_llm_mmlu.py:399-407) all batches are materialised on the device before the
timed steps, and the order comes from a precomputed sampler.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m dynamiq_sigcomm_artifact_b200.train.mmlu --model_name llama-1.2b --aggregation_method dynamiQ_mee_5bit
"""
from __future__ import annotations

import argparse
import os
import time

import torch
import torch.distributed as dist

from ..utils.data import PrecomputedSampler, SyntheticMMLU, gen_orders, mmlu_accuracy
from ..utils.metrics import RunLog
from .engine import TrainConfig, Trainer
from .run import MEASURE_END_STEP, MEASURE_START_STEP, default_lr


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model_name", default="llama-1.2b")
    ap.add_argument("--aggregation_method", default="dynamiQ_aee_5bit")
    ap.add_argument("--per_device_train_batch_size", type=int, default=4)
    ap.add_argument("--block_size", type=int, default=512)
    ap.add_argument("--learning_rate", type=float, default=None)
    ap.add_argument("--max_train_steps", type=int, default=MEASURE_END_STEP + 1)
    ap.add_argument("--eval_items", type=int, default=256)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--output_dir", default=None)
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    use_cuda = torch.cuda.is_available()
    if world > 1:
        if use_cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl" if use_cuda else "gloo")
    rank = dist.get_rank() if dist.is_initialized() else 0
    # the launch scripts use 3e-6 as the MMLU base rate with the causal scaling rule
    lr = args.learning_rate if args.learning_rate is not None else default_lr("causal", world) * 0.3
    cfg = TrainConfig(model=args.model_name, method=args.aggregation_method, micro_batch=args.per_device_train_batch_size,
                      seq_len=args.block_size, lr=lr, total_steps=args.max_train_steps, seed=args.seed,
                      dtype="bf16" if use_cuda else "fp32")
    tr = Trainer(cfg)
    log = RunLog(args.output_dir, rank)
    log.config({**vars(args), "world_size": world, "learning_rate_used": lr})
    vocab = tr.model.config.vocab
    n_train = args.max_train_steps * args.per_device_train_batch_size * world
    data = SyntheticMMLU(vocab, args.block_size, n_train + args.eval_items, seed=args.seed)
    order = gen_orders(n_train, 1, args.seed)[0]
    idx = list(PrecomputedSampler(order, rank, world))
    mb = args.per_device_train_batch_size
    batches = []
    for s in range(args.max_train_steps):  # pre-materialise every batch on the device
        sel = idx[s * mb: (s + 1) * mb]
        ids = torch.stack([data[i][0] for i in sel]).to(tr.device)
        lab = torch.stack([data[i][1] for i in sel]).to(tr.device)
        batches.append((ids, lab))
    t0, measured = None, 0
    for s, (ids, lab) in enumerate(batches):
        if s == MEASURE_START_STEP:
            if use_cuda:
                torch.cuda.synchronize()
            t0 = time.perf_counter()
        # labels are given per position; the model shifts them (position t predicts t + 1)
        loss = float(tr.train_step_device(ids, lab).item())
        if t0 is not None and s < MEASURE_END_STEP:
            measured += 1
        if s % 10 == 0 and rank == 0:
            log.log(f"batch_idx={s} loss={loss:.4f}")
    if t0 is not None:
        if use_cuda:
            torch.cuda.synchronize()
        line = log.results(measured, time.perf_counter() - t0)
        if rank == 0:
            print(line, flush=True)
    # accuracy on held-out items
    tr.model.eval()
    with torch.no_grad():
        ev = range(n_train, n_train + args.eval_items)
        ids = torch.stack([data[i][0] for i in ev]).to(tr.device)
        ans = torch.stack([data[i][2] for i in ev])
        logits = torch.cat([tr.model(ids[i: i + 32])[:, -2].float() for i in range(0, ids.shape[0], 32)])
        acc = mmlu_accuracy(logits, data.answer_tokens, ans)
    if rank == 0:
        log.log(f"mmlu_accuracy={acc:.4f} (chance 0.25)")
    tr.check()
    tr.close()
    if dist.is_initialized():
        dist.destroy_process_group()
    return acc


if __name__ == "__main__":
    main()
