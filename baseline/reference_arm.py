"""Reference arm of bench.py: the unmodified reference code from baseline/_ref.

What runs: the reference's own hook (``P2P_dynamiQ_hook`` chosen by its ``select_hook``), its
``build_comm_state`` and argument defaults (all imported from the copied
``testbed_evaluation/smoke_test_new_comm_hooks.py``), its compressor classes and its
``eden_utils`` CUDA extension built for sm_100, under plain ``DistributedDataParallel`` with
``register_comm_hook([state], hook)`` exactly as that smoke test does (:303-309), around a
random-init Hugging Face model in bf16 with ``torch.optim.AdamW`` and ``LinearLR`` as in
testbed_evaluation/train_llm_causal.py:490-497,614.  None of this package's models, kernels or
engine is imported here.

Two things of the reference cannot run on one 8-GPU host and are replaced by the reference's own
alternatives: its trainer needs a patched ``accelerate`` that is not in the repository
(train_llm_causal.py:16,416), so DDP is constructed directly with the same arguments
(bucket_cap_mb 4000 for DynamiQ, 256 otherwise, :216,:416); and its ring callback needs two
ranks per host plus an RDMA NIC (new_comm_hooks/ring_rdma.py:144-161,445-468), so every hook method
(``dynamiQ_*``, ``bf16``, ``MXfp8``, ``fp4`` / ``fp6``, ``omnireduce``, ``thc``) runs with the ``_butterfly``
suffix and ``BUTTERFLY_RDMA_DISABLE=1``, the reference's own switch to its NCCL point-to-point butterfly
(comm_hooks.py:36-45).

``--method nccl`` (also ``none`` / ``fp32``) is the stock path the reference falls back to when no hook is
selected: plain ``DistributedDataParallel`` with the library all-reduce and 25 MB buckets.

Models: GPT-2 small, the 1.2B Llama-style model and BERT-base (masked LM, 15 % of the positions carry a
label) from ``transformers`` with random-init weights.
"""
from __future__ import annotations

import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
REF_TB = os.path.join(REF, "testbed_evaluation")


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def _hf_model(name: str):
    import torch
    import transformers as tf

    if name == "gpt2-small":
        cfg = tf.GPT2Config(vocab_size=50257, n_positions=1024, n_embd=768, n_layer=12, n_head=12, n_inner=3072)
        return tf.GPT2LMHeadModel(cfg), 50257
    if name == "llama-1.2b":
        cfg = tf.LlamaConfig(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                             num_attention_heads=32, num_key_value_heads=8, max_position_embeddings=2048,
                             rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=True)
        return tf.LlamaForCausalLM(cfg), 128256
    if name == "bert-base":
        cfg = tf.BertConfig(vocab_size=30522, hidden_size=768, num_hidden_layers=12, num_attention_heads=12,
                            intermediate_size=3072, max_position_embeddings=512)
        return tf.BertForMaskedLM(cfg), 30522
    raise ValueError(name)


STOCK = ("nccl", "none", "fp32", "ddp")


def run_reference(args, models) -> None:
    if not os.path.isdir(os.path.join(REF_TB, "new_comm_hooks")):
        return _unavailable("baseline/_ref is missing: run baseline/install_reference.sh <path of the reference checkout>")
    if args.model not in ("gpt2-small", "llama-1.2b", "bert-base"):
        return _unavailable(f"no reference harness for model {args.model}")
    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    method = args.method
    stock = method.lower() in STOCK
    if not stock and "butterfly" not in method.lower():
        method = method + "_butterfly"  # every hook of the reference takes its topology callback from the name
    os.environ["BUTTERFLY_RDMA_DISABLE"] = "1"
    if world > 1 and not stock and world & (world - 1):
        return _unavailable("the reference's butterfly needs a power-of-two world size")
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    mb, seq, _task, desc = models[args.model]
    torch.manual_seed(0)
    model, vocab = _hf_model(args.model)
    model = model.to(torch.bfloat16).to(dev)  # the reference loads torch_dtype=bfloat16
    state = None
    mlm = args.model == "bert-base"
    if world > 1 and stock:
        net = DDP(model, device_ids=[local_rank], bucket_cap_mb=25)
    elif world > 1:
        sys.path.insert(0, REF_TB)
        argv = sys.argv
        sys.argv = ["smoke_test_new_comm_hooks.py", "--aggregation_method", method]
        try:
            import smoke_test_new_comm_hooks as ref_smoke  # the reference's own module, unmodified

            ref_args = ref_smoke.parse_args()
        finally:
            sys.argv = argv
        ref_args.numel = sum(p.numel() for p in model.parameters())
        state = ref_smoke.build_comm_state(ref_args, world)
        hook = ref_smoke.select_hook(method)
        cap = 4000 if "dynamiq" in method.lower() else 256
        dist._DEFAULT_FIRST_BUCKET_BYTES = cap * 1024 * 1024
        net = DDP(model, device_ids=[local_rank], bucket_cap_mb=cap)
        net.register_comm_hook([state], hook)
    else:
        net = model
    opt = torch.optim.AdamW(model.parameters(), lr=1e-5)
    sched = torch.optim.lr_scheduler.LinearLR(opt, start_factor=1.0, end_factor=0.0, total_iters=10_000)

    def batch(i):
        g = torch.Generator().manual_seed(7919 * 0 + 104729 * rank + i)
        return torch.randint(0, vocab, (mb, seq), generator=g, dtype=torch.int64).pin_memory()

    def mlm_labels(ids):  # 15 % of the positions carry a label (80 % [MASK] id 103, 10 % random, 10 % kept)
        g = torch.Generator(device=ids.device).manual_seed(int(ids[0, 0]))
        r = torch.rand(ids.shape, generator=g, device=ids.device)
        sel = r < 0.15
        labels = torch.where(sel, ids, torch.full_like(ids, -100))
        x = ids.clone()
        x[sel & (r < 0.12)] = 103
        rnd = sel & (r >= 0.12) & (r < 0.135)
        x[rnd] = torch.randint(0, vocab, (int(rnd.sum()),), generator=g, device=ids.device)
        return x, labels

    host = [batch(i) for i in range(4)]
    devb = [b.to(dev) for b in host]
    step_idx = [-1]

    def step(ids):
        step_idx[0] += 1
        if state is not None:
            state["batch_idx"] = step_idx[0]
        if mlm:
            x, labels = mlm_labels(ids)
            out = net(input_ids=x, labels=labels)
        else:
            out = net(input_ids=ids, labels=ids)
        out.loss.backward()
        opt.step()
        sched.step()
        opt.zero_grad()
        return out.loss.detach()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    try:
        for i in range(warm):
            float(step(host[i % 4].to(dev, non_blocking=True)).item())
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            step(devb[i % 4])
        e1.record()
        barrier()
        ms_dev = e0.elapsed_time(e1)
        t0 = time.perf_counter()
        for i in range(args.steps):
            last = float(step(host[i % 4].to(dev, non_blocking=True)).item())
        barrier()
        ms_e2e = (time.perf_counter() - t0) * 1e3
    except RuntimeError as e:
        # an exception raised by the reference's own code on this configuration (every rank raises the same one,
        # on the host, inside the hook): reported instead of a number
        why = [ln.strip() for ln in str(e).strip().splitlines() if ln.strip()]
        _unavailable(f"the reference's {method} hook raised on {args.model} at {world} GPUs: " + " | ".join(why[:2])[:300])
        return
    t = torch.tensor([ms_dev, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = float(t[0]), float(t[1])
    tokens = mb * seq * world * args.steps
    if rank == 0:
        print(json.dumps({
            "impl": "reference", "metric": "train_tokens_per_sec", "value": tokens / (ms_dev / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
            "config": {"model": args.model, "arch": desc, "global_batch": mb * world, "seq_len": seq,
                       "parallelism": f"dp{world}", "method": method if world > 1 else "none (1 GPU)",
                       "hook": ("stock DistributedDataParallel, library all-reduce, no hook" if stock or world == 1 else
                                f"reference {hook.__name__} + eden_utils (sm_100 build), NCCL point-to-point butterfly"),
                       "model_impl": "transformers (random init, bf16 parameters), torch.optim.AdamW"},
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": host[0].numel() * 8, "d2h_bytes_per_step": 4},
            "final_loss": last}), flush=True)
    if world > 1:
        dist.destroy_process_group()
