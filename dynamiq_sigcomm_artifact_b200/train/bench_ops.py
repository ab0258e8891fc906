"""Throughput of the model-side and codec-side kernels on training-sized shapes, one GPU.

    python -m dynamiq_sigcomm_artifact_b200.train.bench_ops [--iters 20]

Each operator is timed with CUDA events after warm-up, with a write larger than L2 between
iterations; the line gives the algorithmic bytes, the achieved bandwidth and its fraction of the
measured HBM copy bandwidth (MEASURED_PEAKS.json, or the fallback 6650 GB/s).
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import ops as _ops
from ..ops.layers import FusedAdamW
from .bench_allreduce import HBM_GBS_FALLBACK, measured_peaks


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--only", default="", help="comma list of substrings: time only the kernels whose name has one "
                    "(a profiler capture of one kernel then runs a small program)")
    ap.add_argument("--adamw-params", type=int, default=124_000_000)
    args = ap.parse_args(argv)
    only = [t for t in args.only.split(",") if t]
    dq = _ops.require()
    dev = torch.device("cuda", 0)
    hbm = measured_peaks().get("hbm_gbs", HBM_GBS_FALLBACK)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # 256 MB > 126 MB L2
    bf = torch.bfloat16
    rows = args.rows

    def timed(name, fn, nbytes):
        if only and not any(t in name for t in only):
            return
        for _ in range(args.warmup):
            fn()
        total = 0.0
        for _ in range(args.iters):
            flush.zero_()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        ms = total / args.iters
        print(json.dumps({"kernel": name, "ms": ms, "mbytes": nbytes / 1e6, "gbs": nbytes / ms / 1e6,
                          "hbm_fraction_of_measured": nbytes / ms / 1e6 / hbm}), flush=True)

    for H, tag in ((768, "gpt2"), (2048, "llama")):
        x = torch.randn(rows, H, device=dev).to(bf)
        dy = torch.randn(rows, H, device=dev).to(bf)
        w, b = torch.ones(H, device=dev), torch.zeros(H, device=dev)
        rms = tag == "llama"
        y, mean, rstd = dq.norm_fwd(x, w, None if rms else b, 1e-5, rms)
        timed(f"{'rmsnorm' if rms else 'layernorm'}_fwd_{H}", lambda: dq.norm_fwd(x, w, None if rms else b, 1e-5, rms),
              2 * x.numel() * 2)
        timed(f"{'rmsnorm' if rms else 'layernorm'}_bwd_{H}", lambda: dq.norm_bwd(dy, x, w, mean, rstd, rms),
              3 * x.numel() * 2)
    q = torch.randn(4, 2048, 32, 64, device=dev).to(bf)
    from ..ops.layers import rope_tables

    cos, sin = rope_tables(2048, 64, 500000.0, dev)
    timed("rope_4x2048x32x64", lambda: dq.rope(q, cos, sin, False), 2 * q.numel() * 2)
    gu = torch.randn(rows, 2 * 8192, device=dev).to(bf)
    dyo = torch.randn(rows, 8192, device=dev).to(bf)
    timed("swiglu_fwd_8192", lambda: dq.swiglu_fwd(gu), 3 * rows * 8192 * 2)
    timed("swiglu_bwd_8192", lambda: dq.swiglu_bwd(dyo, gu), 5 * rows * 8192 * 2)
    V, Vp = 50257, 50304
    logits = torch.randn(rows, Vp, device=dev).to(bf)
    labels = torch.randint(0, V, (rows,), device=dev)
    lse, _ = dq.ce_fwd(logits, labels, V, -100)
    one = torch.ones(1, device=dev)
    nv = torch.full((1,), float(rows), device=dev)
    timed("cross_entropy_fwd_50304", lambda: dq.ce_fwd(logits, labels, V, -100), rows * Vp * 2)
    work = logits.clone()
    timed("cross_entropy_bwd_50304", lambda: dq.ce_bwd(work, labels, lse, one, nv, V, -100), 2 * rows * Vp * 2)
    if not only or any(t in "adamw_124M_fp32" for t in only):
        p = torch.randn(args.adamw_params, device=dev).requires_grad_(True)
        p.grad = torch.randn_like(p)
        opt = FusedAdamW([p], lr=1e-4)
        opt.step()
        timed("adamw_124M_fp32", lambda: opt.step(), p.numel() * 28)
        del p, opt
    xs = torch.randn(64 << 20, device=dev)
    timed("superchunk_center_64Mi", lambda: dq.superchunk_center(xs, 8), xs.numel() * 8 + xs.numel() // 32)
    bins = torch.randint(0, 16, (64 << 20,), dtype=torch.uint8, device=dev)
    timed("bins_to_bits_4bit_64Mi", lambda: dq.bins_to_bits(bins, 4), bins.numel() * 1.5)
    # bias gradient of a linear layer: column sums of [8192, 3072] bf16; token-row scatter-add of a tied embedding
    dyl = torch.randn(rows, 3072, device=dev).to(bf)
    timed("colsum_8192x3072_bf16", lambda: dq.colsum(dyl, None), dyl.numel() * 2)
    emb_grad = torch.zeros(50304, 768, device=dev)
    tok = torch.randint(0, 50257, (2 * rows,), device=dev)
    tok_rows = torch.randn(2 * rows, 768, device=dev).to(bf)
    timed("scatter_add_rows_16384x768", lambda: dq.scatter_add_rows(emb_grad, tok, tok_rows, 0.5),
          tok_rows.numel() * 2 + 2 * tok_rows.numel() * 4)
    # bit allocation of the superchunk codec: 64 Mi elements = 256 Ki superchunks
    _, stats = dq.superchunk_center(xs, 8)
    nsc = stats.shape[0]
    state = torch.tensor([3.0, 1.0, 0.0, 0.0], dtype=torch.float64, device=dev)
    scores = torch.empty(nsc, device=dev)
    widths = torch.empty(nsc, dtype=torch.uint8, device=dev)
    timed("superchunk_widths_256Ki", lambda: dq.superchunk_widths(stats, state, scores, widths), nsc * 13)
    timed("superchunk_plan_256Ki", lambda: dq.superchunk_plan(widths), nsc * 3)
    sorted_scores = torch.sort(scores).values
    timed("superchunk_bitrate_update_256Ki", lambda: dq.superchunk_bitrate_update(sorted_scores, state, 4.375), nsc * 4)
    # upper levels of a 2^23-point Walsh-Hadamard transform (THC partitions): levels 10..22 in three passes
    v = torch.randn(1 << 23, device=dev)
    timed("fwht_levels_2p23_five_levels", lambda: dq.fwht_levels_(v, 10, 5, 1.0), v.numel() * 8)
    from ..ops.fwht import fwht_pow2

    timed("fwht_pow2_2p23_whole_vector", lambda: fwht_pow2(v), v.numel() * 8 * 4)


if __name__ == "__main__":
    main()
