"""Training engine: model + DDP + comm hook + fused optimizer, one call per step.

The public entry point is :meth:`Trainer.train_step`: it takes a batch of token ids in pinned
host memory, copies it to the device, runs forward, backward (the hook's collectives overlap
it on a side stream), the optimizer, and returns the loss as a Python float.

Reference counterpart: ``train()`` and its set-up in testbed_evaluation/train_llm_causal.py:331-394,
398-646 (HF model in bf16, torch AdamW, LinearLR, DDP through a patched ``accelerate`` with
``bucket_cap_mb=4000`` for DynamiQ so that the whole model is one bucket, :216,:416).  Compute is bf16
autocast over fp32 master weights and fp32 gradient buckets.

Bucket size (``TrainConfig.bucket_cap_mb``, 0 = automatic): every method whose collective is one of this
package's kernels gets ONE bucket for the whole model (4000 MB cap, the reference's setting for DynamiQ); the
library all-reduce methods (``fp32`` / ``none`` / ``nccl``) keep 25 MB buckets, and so does a single-GPU run
(100 MB for the 1.2 B model), where a bucket is only the unit of the AdamW step that runs under backward.  Measured on four B200s: the
collective kernel and the backward GEMMs compete for the same SMs, so a collective that runs under backward
costs its own SM time anyway, and twenty small ones add their fixed latencies on top - GPT-2 small 11.09 ms
per step with 25 MB buckets, 10.74 with 200 MB, 10.64 with one bucket (1 GPU: 10.17); Llama 1.2B 75.2 ms
with 100 MB buckets, 72.9 with one; BERT-base 12.90 -> 12.63 ms.

Two gradient paths (``TrainConfig.reducer``): ``"flat"`` (default) is this package's bucket reducer
(parallel/reducer.py: gradient arena written in place by the backward kernels, communication hook
and the AdamW step of each bucket on a side stream under the rest of backward); ``"ddp"`` wraps the
model in ``DistributedDataParallel`` and registers the same hook through ``register_comm_hook``, as
a user with an existing DDP model would.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

from .. import hooks
from ..config import DynamiqConfig
from ..models import build_model, mask_tokens
from ..ops.layers import FusedAdamW
from ..ops.linear import enable_shadows


def default_bucket_cap_mb(method: str, world: int = 2, model: str = "") -> int:
    """One bucket for the whole model when the collective is this package's own kernel; the library's usual
    25 MB when it is the library's all-reduce (which overlaps backward without taking SMs from it); and small
    buckets on a single GPU, where a bucket is only the unit of the optimizer step that runs under backward."""
    from ..config import parse_method

    if world <= 1:
        return 100 if "1.2b" in model else 25
    return 25 if parse_method(method).hook in ("fp32", "fp16") else 4000


@dataclass
class TrainConfig:
    model: str = "gpt2-small"
    method: str = "dynamiQ_aee_5bit"
    micro_batch: int = 8
    seq_len: int = 1024
    lr: float = 1e-5
    weight_decay: float = 0.0
    total_steps: int = 10_000
    bucket_cap_mb: int = 0  # 0: automatic (see the module docstring)
    tail_pipeline_mb: int = 0  # > 0 ("flat" reducer on CUDA): buckets of this size, all sent AFTER backward, each
    #                            bucket's optimizer step on a second stream under the next bucket's collective
    seed: int = 0
    dtype: str = "bf16"  # autocast dtype; parameters, gradients and optimizer state are fp32
    task: str = "causal"  # causal | mlm
    topology: Optional[str] = None
    comm_ctas: int = 64
    comm_threads: int = 256
    tail_ctas: int = 148  # grid of the step's last bucket (nothing left to overlap)
    comm_prefetch: bool = True  # staging buffer of the collective kernel (off: half the shared memory per CTA)
    warmup_steps: int = 2
    measure_comm_error: bool = False
    cuda_graphs: bool = True  # capture each transformer block's forward and backward as CUDA graphs
    reducer: str = "flat"  # "flat": gradient arena + bucket pipeline of this package; "ddp": torch DDP + comm hook
    sparse_embedding: Optional[bool] = None  # True: tied-embedding lookup gradient exchanged as token rows


class Trainer:
    def __init__(self, cfg: TrainConfig, device: Optional[torch.device] = None):
        self.cfg = cfg
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        if device is None:
            device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if torch.cuda.is_available() \
                else torch.device("cpu")
        self.device = device
        torch.manual_seed(cfg.seed)  # identical initial weights on every rank
        self.model = build_model(cfg.model).to(device)
        # bf16 working copies of the linear weights, kept in step by the optimizer kernel
        self.shadows = enable_shadows(self.model) if (device.type == "cuda" and cfg.dtype == "bf16") else {}
        self.graphed = False
        self.state = None
        self.ddp = None
        self.reducer = None
        self.net = self.model
        self.opt = FusedAdamW(self.model.parameters(), lr=cfg.lr, weight_decay=cfg.weight_decay, shadows=self.shadows)
        if cfg.reducer not in ("flat", "ddp"):
            raise ValueError(f"unknown reducer {cfg.reducer!r}")
        if cfg.bucket_cap_mb <= 0:
            cfg.bucket_cap_mb = default_bucket_cap_mb(cfg.method, self.world, cfg.model)
        dcfg = None
        if self.world > 1:
            dcfg = DynamiqConfig.from_env(method=cfg.method, seed=cfg.seed, topology=cfg.topology,
                                          comm_ctas=cfg.comm_ctas, comm_threads=cfg.comm_threads, tail_ctas=cfg.tail_ctas,
                                          comm_prefetch=cfg.comm_prefetch,
                                          warmup_steps=cfg.warmup_steps, measure_comm_error=cfg.measure_comm_error)
        use_graphs = cfg.cuda_graphs and device.type == "cuda" and cfg.dtype == "bf16"
        if cfg.reducer == "flat":
            from ..parallel.reducer import BucketReducer

            hook = state_list = None
            if dcfg is not None:
                state_list = hooks.build_comm_state(dcfg)
                hook = hooks.select_comm_hook(cfg.method, dcfg.topology)
                self.state = state_list[0]
            # the arena has to exist before the blocks are captured: the graphs keep its addresses
            defer = cfg.tail_pipeline_mb > 0 and device.type == "cuda"
            self.reducer = BucketReducer(self.model, cfg.tail_pipeline_mb if defer else cfg.bucket_cap_mb, hook, state_list,
                                         defer=defer,
                                         on_reduced=lambda bi, ps: self.opt.step_params(bi, ps),
                                         direct=(device.type == "cuda" and cfg.dtype == "bf16"), install=False,
                                         sparse_embedding=cfg.sparse_embedding)
            if self.world > 1:
                self.reducer.broadcast_parameters(0)
                if self.shadows:
                    enable_shadows(self.model)
            if use_graphs:
                self.graphed = self._graph_blocks()
            self.reducer.arena.zero_()
            self.reducer.install_marks()
            self.opt._opt_called = True  # the scheduler's "step() before optimizer.step()" check
        else:
            if use_graphs:
                self.graphed = self._graph_blocks()
            if self.world > 1:
                self.ddp = DDP(self.model, device_ids=[device.index] if device.type == "cuda" else None,
                               bucket_cap_mb=cfg.bucket_cap_mb, gradient_as_bucket_view=True, broadcast_buffers=False)
                self.state = hooks.register(self.ddp, cfg.method, config=dcfg)
                self.net = self.ddp
            else:
                self._flatten_grads()
        self.sched = torch.optim.lr_scheduler.LinearLR(self.opt, start_factor=1.0, end_factor=0.0,
                                                       total_iters=cfg.total_steps)
        self.step_idx = 0
        self._dev_ids = None
        self._status_host = None  # pinned copy of the collective engine's status words, refreshed every step
        self._status_event = None
        self._gen = torch.Generator(device=device).manual_seed(cfg.seed + 17 * self.rank + 1) \
            if device.type == "cuda" else torch.Generator().manual_seed(cfg.seed + 17 * self.rank + 1)
        self.autocast_dtype = {"bf16": torch.bfloat16, "fp32": None}[cfg.dtype]

    def _graph_blocks(self) -> bool:
        """Capture every transformer block (forward and backward) as CUDA graphs: a step then issues
        two graph launches per block instead of ~100 eager kernels, which takes the host off the
        critical path.  Shapes are fixed by (micro_batch, seq_len); evaluation runs eagerly.  DDP's
        parameter hooks still fire block by block, so bucket collectives keep overlapping backward."""
        m, cfg = self.model, self.cfg
        blocks = getattr(m, "blocks", None) or getattr(m, "layers", None)
        if blocks is None:
            return False
        c = m.config
        hidden = getattr(c, "d_model", None) or getattr(c, "hidden")
        x = torch.randn(cfg.micro_batch, cfg.seq_len, hidden, device=self.device, dtype=torch.bfloat16,
                        requires_grad=True)
        if hasattr(m, "_tables"):
            cos, sin = m._tables(cfg.seq_len, self.device)
            sample = tuple((x.detach().clone().requires_grad_(True), cos, sin) for _ in blocks)
        else:
            sample = tuple((x.detach().clone().requires_grad_(True),) for _ in blocks)
        import warnings

        from ..utils import counters

        # kernels of this package launched by one forward + backward of a block (replays repeat them)
        before = counters.total()
        with torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=False):
            blocks[0](*sample[0]).float().sum().backward()
        self._launches_per_graphed_step = (counters.total() - before) * len(blocks)
        # parameters were created on the default stream and the capture runs on a side stream
        warnings.filterwarnings("ignore", message="The AccumulateGrad node's stream does not match")
        try:
            with torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=False):
                # with a gradient arena the blocks write their parameter gradients in place and
                # autograd sees none for them
                graphed = torch.cuda.make_graphed_callables(tuple(blocks), sample, num_warmup_iters=3,
                                                            allow_unused_input=self.reducer is not None)
        except Exception as e:  # fall back to eager execution, loudly
            print(f"[dynamiq] CUDA graph capture of the blocks failed ({type(e).__name__}: {e}); running eagerly",
                  flush=True)
            return False
        for i, g in enumerate(graphed):
            blocks[i] = g
        if self.reducer is None:
            for p in m.parameters():  # capture warm-up ran backward passes: drop their gradients
                p.grad = None
        return True

    def _flatten_grads(self) -> None:
        """Single-process runs: all gradients live in one flat buffer, zeroed by one memset."""
        params = [p for p in self.model.parameters() if p.requires_grad]
        total = sum(p.numel() for p in params)
        self._flat_grad = torch.zeros(total, dtype=torch.float32, device=self.device)
        off = 0
        for p in params:
            p.grad = self._flat_grad[off: off + p.numel()].view_as(p)
            off += p.numel()

    # -- one step ------------------------------------------------------------------------
    def train_step_device(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One optimizer step on device-resident token ids; returns the loss tensor (no sync)."""
        cfg = self.cfg
        if self.state is not None:
            self.state.begin_step(self.step_idx)
        if cfg.task == "mlm" and labels is None:
            c = self.model.config
            input_ids, labels = mask_tokens(input_ids, c.vocab, c.mask_token_id, self._gen)
        elif labels is None:
            labels = input_ids
        if self.autocast_dtype is not None and self.device.type == "cuda":
            with torch.autocast("cuda", dtype=self.autocast_dtype):
                loss = self.net(input_ids, labels)
        else:
            loss = self.net(input_ids, labels)
        if self.reducer is not None:
            self.opt.advance()
            self.reducer.begin_step()
        loss.backward()
        if self.graphed:
            from ..utils import counters

            counters.add("graphed_blocks", self._launches_per_graphed_step)
        if self.reducer is not None:
            self.reducer.finish()  # every bucket: hook, then its AdamW step, on the side stream
            self.sched.step()
        else:
            self.opt.step()
            self.sched.step()
            if self.ddp is None:
                self._flat_grad.zero_()
            else:
                self.opt.zero_grad(set_to_none=False)
        self.step_idx += 1
        self._poll_status(enqueue=True)
        return loss.detach()

    def train_step(self, input_ids_host: torch.Tensor, labels_host: Optional[torch.Tensor] = None) -> float:
        """Public API: host batch in, loss out.  Copies the batch to the device every call."""
        ids = input_ids_host.to(self.device, non_blocking=True)
        lab = labels_host.to(self.device, non_blocking=True) if labels_host is not None else None
        loss = float(self.train_step_device(ids, lab).item())
        self._poll_status(enqueue=False)  # the loss read-back synchronised: this step's status copy has landed
        return loss

    def _poll_status(self, enqueue: bool) -> None:
        """A device-side wait that gave up leaves an error code in the engine's status words and a partly
        reduced bucket behind.  Every step queues a 16-byte copy of those words into pinned memory behind the
        step's kernels; the copy of the previous step (or of this one, once the caller has synchronised) is
        inspected without blocking, so a failed collective raises :class:`CollectiveTimeout` at most one step
        late instead of at the end of the run.  A rank whose peer gave up runs out of its own wait budget in
        the same collective, so every rank raises."""
        eng = self.state["engine"] if self.state is not None else None
        if eng is None or self.device.type != "cuda":
            return
        if self._status_event is not None and self._status_event.query():
            from ..parallel.fused import CollectiveTimeout, decode_status

            msg = decode_status(self._status_host.tolist())
            self._status_event = None
            if msg is not None:
                raise CollectiveTimeout(f"rank {self.rank}: {msg} (noticed at step {self.step_idx})")
        if enqueue:
            if self._status_host is None:
                self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
            self._status_host.copy_(eng._status_view, non_blocking=True)
            self._status_event = torch.cuda.Event()
            self._status_event.record()

    def tokens_per_step(self) -> int:
        return self.cfg.micro_batch * self.cfg.seq_len * self.world

    def synthetic_batch(self, pinned: bool = True) -> torch.Tensor:
        """Token ids uniform in [0, vocab) from a seeded generator, in (pinned) host memory."""
        g = torch.Generator().manual_seed(self.cfg.seed * 7919 + self.rank * 104729 + self.step_idx)
        c = self.model.config
        ids = torch.randint(0, c.vocab, (self.cfg.micro_batch, self.cfg.seq_len), generator=g, dtype=torch.int64)
        return ids.pin_memory() if pinned and torch.cuda.is_available() else ids

    def check(self) -> None:
        """Blocking check of the collective engine's status (call before saving a checkpoint or reporting
        results)."""
        if self.state is not None and self.state["engine"] is not None:
            self.state["engine"].check()

    def close(self) -> None:
        if self.state is not None:
            self.state.close()
