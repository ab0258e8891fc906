"""Gradient arena + bucket reducer: the trainer's own replacement for DDP's reducer.

DDP's reducer (which the reference drives through ``register_comm_hook``,
testbed_evaluation/train_llm_causal.py:398-425 and new_comm_hooks/comm_hooks.py) allocates its
own buckets, learns readiness from per-parameter autograd hooks and leaves the optimizer for after
the backward pass.  On one B200 that costs, per parameter and step: a memset and an accumulate
kernel for the gradient (16 bytes of HBM traffic), an optimizer pass that nothing overlaps
(30 bytes), and a Python hook.  This reducer is built around fixed addresses instead:

* **Arena.**  All gradients live in one flat fp32 buffer laid out in the order in which they become
  ready during backward (head, last block ... first block, embeddings); a bucket is a contiguous
  slice of whole groups.  ``param.grad`` is a view; ``param._dq_grad`` is the same view for modules
  whose backward writes it in place (``MasterLinear``, ``LayerNorm`` / ``RMSNorm``, ``TiedEmbedding``):
  those never allocate, zero or accumulate a gradient, and CUDA graphs of the blocks can bake the
  addresses in.  Other parameters accumulate through autograd as usual and are zeroed after use.
* **Readiness.**  An identity autograd node in front of every block reports "everything after me is
  done" when backward reaches it; the rest is flushed when backward returns.
* **Pipeline.**  A ready bucket goes to the side stream: communication hook (same contract as a DDP
  comm hook: ``hook(state, bucket) -> Future[Tensor]``, the bucket being a ``FlatBucket``), then the
  fused AdamW step of exactly that bucket's parameters, both overlapping the rest of backward.
  Without gradient clipping nothing needs the whole gradient before the first update.

* **Tied embedding across ranks** (``sparse_embedding=True``; off by default):
  the dense part of a tied embedding's gradient (the output projection's weight gradient) exists at the very
  start of backward, the lookup part only at its end but touches at most one row per token.  The parameter is
  therefore bucketed with the head (reduced through the hook under the whole backward pass); the lookup part
  travels as token rows (all-gather of ids and bf16 rows) and every rank adds all ranks' rows in the same
  order after the dense part has been reduced, followed by that parameter's AdamW step.  This removes the
  compressed collective of a vocabulary-sized bucket from the step's tail, but on B200 it measured slower than
  the dense path (GPT-2 small, 2 GPUs: 10.77 vs 10.61 ms per step; Llama 1.2B: 74.4 vs 73.2 ms): the collective
  kernel and the GEMMs of backward compete for the same SMs, so moving the big collective under backward
  costs as much as it saves, and the row exchange adds two library all-gathers and a sort.

In this mode one backward pass per step is assumed (a second one overwrites the in-place
gradients); accumulate micro-batches with ``direct=False``.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

ALIGN = 4  # elements: 16-byte aligned views for vector loads and GEMM outputs


class FlatBucket:
    """What a communication hook sees: the subset of ``dist.GradBucket`` the hooks use."""

    def __init__(self, index: int, buffer: torch.Tensor, params: List[nn.Parameter], last: bool):
        self._index, self._buffer, self._params, self._last = index, buffer, params, last
        self.exposed = last  # True when nothing of backward runs beside this bucket's collective (wide grid)

    def index(self) -> int:
        return self._index

    def buffer(self) -> torch.Tensor:
        return self._buffer

    def gradients(self) -> List[torch.Tensor]:
        return [p.grad for p in self._params]

    def parameters(self) -> List[nn.Parameter]:
        return list(self._params)

    def is_last(self) -> bool:
        return self._last

    def set_buffer(self, t: torch.Tensor) -> None:
        if t.data_ptr() != self._buffer.data_ptr():
            self._buffer.copy_(t.reshape(-1))


class _Mark(torch.autograd.Function):
    """Identity whose backward calls `cb()`: placed on a block's input, it fires once the block's
    backward (and everything behind it) has been issued."""

    @staticmethod
    def forward(ctx, x, cb):
        ctx.cb = cb
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.cb()
        return g, None


def direct_modules():
    from ..ops.embedding import TiedEmbedding
    from ..ops.layers import LayerNorm, RMSNorm
    from ..ops.linear import MasterLinear

    return (MasterLinear, LayerNorm, RMSNorm, TiedEmbedding)


def find_blocks(model: nn.Module) -> Optional[nn.ModuleList]:
    for name in ("blocks", "layers"):
        b = getattr(model, name, None)
        if isinstance(b, nn.ModuleList) and len(b) > 0:
            return b
    return None


class BucketReducer:
    """See the module docstring.  `hook` / `hook_state` may be None (single process): buckets then go
    straight to `on_reduced`."""

    def __init__(self, model: nn.Module, bucket_cap_mb: float = 25.0, hook: Optional[Callable] = None,
                 hook_state=None, on_reduced: Optional[Callable[[int, List[nn.Parameter]], None]] = None,
                 direct: bool = True, side_stream: bool = True, group=None, install: bool = True,
                 sparse_embedding: Optional[bool] = None, defer: bool = False):
        """`defer`: no bucket is sent while backward runs; after it, the buckets go out back to back on the side
        stream and every bucket's consumer (`on_reduced`, the optimizer step) runs on a second stream as soon as
        its bucket is reduced - bucket k's optimizer step overlaps bucket k+1's collective instead of backward."""
        self.model, self.hook, self.hook_state, self.on_reduced = model, hook, hook_state, on_reduced
        self.defer = bool(defer)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._sparse_wanted = sparse_embedding
        params = [p for p in model.parameters() if p.requires_grad]
        if not params:
            raise ValueError("model has no trainable parameters")
        self.device = params[0].device
        self.cuda = self.device.type == "cuda"
        self.direct = bool(direct and self.cuda)
        self.blocks = find_blocks(model)
        # tied embeddings whose lookup gradient is exchanged as rows (needs the in-place gradient path)
        want = bool(self._sparse_wanted)  # off unless asked for: measured slower than the dense path (see docstring)
        self.sparse_params: List[nn.Parameter] = []
        if want and self.direct and self.blocks is not None:
            from ..ops.embedding import TiedEmbedding

            self.sparse_params = [m.weight for m in model.modules() if isinstance(m, TiedEmbedding)
                                  and m.weight.requires_grad]
        self._sparse_ids = {id(p) for p in self.sparse_params}
        self.groups = self._make_groups(params)
        self._layout(bucket_cap_mb)
        self.side = torch.cuda.Stream(self.device) if (self.cuda and side_stream) else None
        self.consumer_stream = torch.cuda.Stream(self.device) if (self.side is not None and self.defer) else None
        self._pending: List[int] = []
        if self.defer:
            for b in self.buckets:
                b.exposed = True
        self._ready_upto = -1  # groups [0, _ready_upto] have been reported
        self._next_bucket = 0
        self._handles = []
        if install:
            self.install_marks()
        self.launched = 0

    # -- construction ---------------------------------------------------------------------
    def _make_groups(self, params: Sequence[nn.Parameter]) -> List[List[nn.Parameter]]:
        """Groups in the order they become ready: [after-the-blocks + last block], ..., block 0, [before]."""
        if self.blocks is None:
            return [list(params)]
        in_block: Dict[int, int] = {}
        for i, b in enumerate(self.blocks):
            for p in b.parameters():
                in_block[id(p)] = i
        pre, post, per_block = [], [], [[] for _ in self.blocks]
        seen_block = False
        for p in params:
            bi = in_block.get(id(p))
            if bi is not None:
                per_block[bi].append(p)
                seen_block = True
            elif id(p) in self._sparse_ids:
                post.insert(0, p)  # its dense gradient (output projection) is the first thing backward produces
            elif seen_block:
                post.append(p)
            else:
                pre.append(p)
        n = len(self.blocks)
        groups = [post + per_block[-1]] + [per_block[i] for i in range(n - 2, -1, -1)] + [pre]
        # an empty group reports together with the previous non-empty one
        keep, remap = [], {}
        for gi, g in enumerate(groups):
            if g:
                keep.append(g)
            remap[gi] = max(len(keep) - 1, 0)
        self._group_of_block = {b: remap[n - 1 - b] for b in range(n)}
        return keep

    def _layout(self, cap_mb: float) -> None:
        direct_ids = set()
        if self.direct:
            kinds = direct_modules()
            for m in self.model.modules():
                if isinstance(m, kinds):
                    for p in m.parameters(recurse=False):
                        direct_ids.add(id(p))
        cap = max(1, int(cap_mb * 1024 * 1024 // 4))
        # buckets: whole groups, closed when they reach the cap
        self.bucket_groups: List[List[int]] = []
        cur, cur_n = [], 0
        for gi, g in enumerate(self.groups):
            cur.append(gi)
            cur_n += sum(p.numel() for p in g)
            if cur_n >= cap:
                self.bucket_groups.append(cur)
                cur, cur_n = [], 0
        if cur:
            self.bucket_groups.append(cur)
        off = 0
        spans, slots, gaps = [], {}, []
        for groups in self.bucket_groups:
            start = off
            for gi in groups:
                for p in self.groups[gi]:
                    n = p.numel()
                    padded = getattr(p, "_dq_padded_shape", None) if id(p) in direct_ids else None
                    reserve = max(n, padded[0] * padded[1]) if padded else n
                    aligned = (reserve + ALIGN - 1) // ALIGN * ALIGN
                    slots[id(p)] = (off, n, padded)
                    if aligned > reserve:
                        gaps.append((off + reserve, aligned - reserve))
                    off += aligned
            spans.append((start, off))
        self.arena = torch.zeros(off, dtype=torch.float32, device=self.device)
        self.spans = spans
        self._gap_index = None
        if gaps:
            self._gap_index = torch.cat([torch.arange(s, s + n) for s, n in gaps]).to(self.device)
        self.bucket_params: List[List[nn.Parameter]] = []
        self.bucket_accum: List[List[nn.Parameter]] = []  # parameters whose gradients autograd accumulates
        self.group_bucket = {}
        for bi, groups in enumerate(self.bucket_groups):
            ps = [p for gi in groups for p in self.groups[gi]]
            self.bucket_params.append(ps)
            self.bucket_accum.append([p for p in ps if id(p) not in direct_ids])
            for gi in groups:
                self.group_bucket[gi] = bi
        for p in (q for ps in self.bucket_params for q in ps):
            o, n, padded = slots[id(p)]
            p.grad = self.arena[o: o + n].view_as(p)
            if id(p) in direct_ids:
                p._dq_grad = p.grad
                if padded:
                    p._dq_grad_padded = self.arena[o: o + padded[0] * padded[1]].view(padded)
            if id(p) in self._sparse_ids:
                p._dq_sparse = {"ids": None, "rows": None}
        self.buckets = [FlatBucket(bi, self.arena[s:e], self.bucket_params[bi], bi == len(spans) - 1)
                        for bi, (s, e) in enumerate(spans)]
        self.n_direct = len(direct_ids)
        # announce the largest bucket to the hook state, so that the collective engine is sized once, before
        # the first step, for exactly this arena
        st = self.hook_state[0] if isinstance(self.hook_state, (list, tuple)) and self.hook_state else self.hook_state
        if isinstance(st, dict):
            st["max_bucket_numel"] = max([e - s0 for s0, e in spans] + [int(st.get("max_bucket_numel", 0))])

    def install_marks(self) -> None:
        """Put the readiness markers in front of the blocks (after any CUDA-graph capture of them)."""
        if self.blocks is None or self._handles:
            return
        for bi, blk in enumerate(self.blocks):
            gi = self._group_of_block[bi]

            def pre(mod, args, _gi=gi):
                x = args[0]
                if torch.is_grad_enabled() and isinstance(x, torch.Tensor) and x.requires_grad:
                    return (_Mark.apply(x, lambda: self.group_ready(_gi)),) + tuple(args[1:])
                return None

            self._handles.append(blk.register_forward_pre_hook(pre))

    def detach(self) -> None:
        """Remove the hooks and the in-place gradient views (gradients stay where they are)."""
        for h in self._handles:
            h.remove()
        self._handles = []
        for ps in self.bucket_params:
            for p in ps:
                for a in ("_dq_grad", "_dq_grad_padded", "_dq_sparse"):
                    if hasattr(p, a):
                        delattr(p, a)

    # -- one step -------------------------------------------------------------------------
    def begin_step(self) -> None:
        self._ready_upto = -1
        self._next_bucket = 0
        self._pending = []

    def group_ready(self, gi: int) -> None:
        """Groups are reported in order; reporting group g implies every group before it."""
        if gi <= self._ready_upto:
            return
        self._ready_upto = gi
        while self._next_bucket < len(self.bucket_groups) and self.bucket_groups[self._next_bucket][-1] <= gi:
            self._launch(self._next_bucket)
            self._next_bucket += 1

    def _launch(self, bi: int) -> None:
        if self.defer and self.consumer_stream is not None:
            self._pending.append(bi)  # sent by finish(), after backward
            return
        bucket = self.buckets[bi]
        self.launched += 1
        if self.side is not None:
            self.side.wait_stream(torch.cuda.current_stream(self.device))
            ctx = torch.cuda.stream(self.side)
        else:
            import contextlib

            ctx = contextlib.nullcontext()
        with ctx, torch.no_grad():
            if self.hook is not None:
                fut = self.hook(self.hook_state, bucket)
                fut.wait()
                bucket.set_buffer(fut.value())
            if self._gap_index is not None and bucket.is_last():
                self.arena.index_fill_(0, self._gap_index, 0.0)
            if self.on_reduced is not None:  # the consumer (optimizer) runs here, so the gradients are spent
                ready = [p for p in self.bucket_params[bi] if id(p) not in self._sparse_ids]
                self.on_reduced(bi, ready)
                for p in self.bucket_accum[bi]:
                    p.grad.zero_()

    def finish(self) -> None:
        """After ``loss.backward()``: flush what no marker reported and join the side stream."""
        self.group_ready(len(self.groups) - 1)
        if self._pending:
            self._run_deferred()
        if self.sparse_params:
            self._finish_sparse()
        if self.side is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.side)

    def _run_deferred(self) -> None:
        """Every bucket's hook on the side stream, back to back; its consumer on a second stream behind an event."""
        cur = torch.cuda.current_stream(self.device)
        self.side.wait_stream(cur)
        self.consumer_stream.wait_stream(cur)
        for bi in self._pending:
            bucket = self.buckets[bi]
            self.launched += 1
            with torch.cuda.stream(self.side), torch.no_grad():
                if self.hook is not None:
                    fut = self.hook(self.hook_state, bucket)
                    fut.wait()
                    bucket.set_buffer(fut.value())
                if self._gap_index is not None and bucket.is_last():
                    self.arena.index_fill_(0, self._gap_index, 0.0)
                reduced = torch.cuda.Event()
                reduced.record(self.side)
            if self.on_reduced is not None:
                with torch.cuda.stream(self.consumer_stream), torch.no_grad():
                    self.consumer_stream.wait_event(reduced)
                    ready = [p for p in self.bucket_params[bi] if id(p) not in self._sparse_ids]
                    self.on_reduced(bi, ready)
                    for p in self.bucket_accum[bi]:
                        p.grad.zero_()
        self._pending = []
        self.side.wait_stream(self.consumer_stream)  # finish() joins the side stream

    def _finish_sparse(self) -> None:
        """Exchange the lookup rows of the tied embeddings, add every rank's rows (same order everywhere), then
        hand the parameters to the consumer."""
        from .. import ops as _ops
        from ..utils import counters

        dq = _ops.require()
        stream = self.side if self.side is not None else torch.cuda.current_stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream), torch.no_grad():
            for p in self.sparse_params:
                sp = p._dq_sparse
                ids, rows = sp["ids"], sp["rows"]
                if ids is None:
                    raise RuntimeError("a tied embedding took no part in this backward pass")
                if self.world > 1:
                    all_ids = torch.empty(self.world * ids.numel(), dtype=ids.dtype, device=ids.device)
                    all_rows = torch.empty(self.world * rows.shape[0], rows.shape[1], dtype=rows.dtype, device=rows.device)
                    dist.all_gather_into_tensor(all_ids, ids.contiguous(), group=self.group)
                    dist.all_gather_into_tensor(all_rows, rows, group=self.group)
                else:
                    all_ids, all_rows = ids.contiguous(), rows
                dq.scatter_add_rows(p.grad, all_ids, all_rows, 1.0 / self.world)
                counters.add("scatter_add_rows")
                sp["ids"] = sp["rows"] = None
                ids.record_stream(stream)
                rows.record_stream(stream)
            if self.on_reduced is not None:
                self.on_reduced(-1, self.sparse_params)

    def zero_accumulated(self) -> None:
        """Without `on_reduced`: call after the optimizer step (in-place gradients need no zeroing)."""
        for ps in self.bucket_accum:
            for p in ps:
                p.grad.zero_()

    # -- helpers --------------------------------------------------------------------------
    def broadcast_parameters(self, src: int = 0) -> None:
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            with torch.no_grad():
                for t in list(self.model.parameters()) + list(self.model.buffers()):
                    dist.broadcast(t.data, src, group=self.group)

    def describe(self) -> dict:
        return {"buckets": len(self.buckets), "arena_elements": int(self.arena.numel()),
                "bucket_elements": [e - s for s, e in self.spans], "direct_parameters": self.n_direct,
                "accumulated_parameters": sum(len(a) for a in self.bucket_accum)}
