"""Single-GPU driver that launches each hand-written kernel once or a few times on a case
larger than L2 and a few hundred MB at most: the form used for profiler captures, and a
quick event-timed bandwidth / throughput read-out without a profiler.

  python bench/probe_kernels.py --what ag_emulated      two virtual ranks, fused all-gather + GEMM
  python bench/probe_kernels.py --what rs_emulated      two virtual ranks, fused GEMM + reduce-scatter
  python bench/probe_kernels.py --what ar_emulated      two virtual ranks, fused GEMM + two-shot all-reduce
  python bench/probe_kernels.py --what moe              metadata + dispatch + combine (one rank)
  python bench/probe_kernels.py --what swiglu           stand-alone SwiGLU
  python bench/probe_kernels.py --what all

The multi-rank protocols run as ONE cooperative launch over both virtual ranks' data
(kernels that wait on one another are never separate launches on one GPU).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def timed(fn, iters):
    import torch
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="all")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--pairs", type=int, default=1, help="1: the virtual ranks run CTA pairs with 512-row tiles "
                    "(the production tile shape), 0: single-CTA 128 x 256 tiles")
    args = ap.parse_args()
    os.environ["TRIDIST_EMU_PAIR"] = str(args.pairs)
    import torch
    from tridist_b200.parallel.runtime import EmulatedWorld, ProcessWorld
    from tridist_b200.utils.roofline import load_peaks
    peaks = load_peaks()
    dt = torch.bfloat16
    what = args.what

    if what in ("ag_emulated", "all"):
        from tridist_b200.ops.all_gather_gemm import ag_gemm_emulated, create_ag_gemm_intra_node_context
        R, m_pr, K, n_pr = 2, 2048, 8192, 4096
        w = EmulatedWorld(R)
        ctxs = [create_ag_gemm_intra_node_context(m_pr * R, K, dt, dt, r, R, M_PER_CHUNK=m_pr, world=w) for r in range(R)]
        a = [(torch.randn(m_pr, K, device="cuda") * 0.05).to(dt) for _ in range(R)]
        b = [(torch.randn(n_pr, K, device="cuda") * 0.05).to(dt) for _ in range(R)]
        c = [torch.empty(m_pr * R, n_pr, dtype=dt, device="cuda") for _ in range(R)]
        ms = timed(lambda: ag_gemm_emulated(ctxs, a, b, c), args.iters)
        w.check(sync=True)
        flops = R * 2.0 * (m_pr * R) * n_pr * K
        print(json.dumps({"kernel": "fused_gemm_kernel (AG, 2 virtual ranks)", "ms": round(ms, 4),
                          "tflops": round(flops / ms / 1e9, 1)}))

    if what in ("rs_emulated", "all"):
        from tridist_b200.ops.gemm_reduce_scatter import create_gemm_rs_intra_node_context, gemm_rs_emulated
        R, M, N, kl = 2, 4096, 4096, 4096
        w = EmulatedWorld(R)
        ctxs = [create_gemm_rs_intra_node_context(M, N, dt, r, R, world=w) for r in range(R)]
        a = [(torch.randn(M, kl, device="cuda") * 0.05).to(dt) for _ in range(R)]
        b = [(torch.randn(N, kl, device="cuda") * 0.05).to(dt) for _ in range(R)]
        ms = timed(lambda: gemm_rs_emulated(ctxs, a, b), args.iters)
        w.check(sync=True)
        flops = R * 2.0 * M * N * kl
        print(json.dumps({"kernel": "fused_gemm_kernel (RS, 2 virtual ranks)", "ms": round(ms, 4),
                          "tflops": round(flops / ms / 1e9, 1)}))

    if what in ("ar_emulated", "all"):
        from tridist_b200.ops.gemm_allreduce import create_gemm_ar_intra_node_context, gemm_ar_emulated
        R, M, N, kl = 2, 4096, 4096, 4096
        w = EmulatedWorld(R)
        ctxs = [create_gemm_ar_intra_node_context(M, N, dt, dt, r, R, M_PER_CHUNK=64, world=w) for r in range(R)]
        a = [(torch.randn(M, kl, device="cuda") * 0.05).to(dt) for _ in range(R)]
        b = [(torch.randn(N, kl, device="cuda") * 0.05).to(dt) for _ in range(R)]
        c = [torch.empty(M, N, dtype=dt, device="cuda") for _ in range(R)]
        ms = timed(lambda: gemm_ar_emulated(ctxs, a, b, c, mode="two_shot"), args.iters)
        w.check(sync=True)
        flops = R * 2.0 * M * N * kl
        print(json.dumps({"kernel": "fused_gemm_kernel (two-shot AR, 2 virtual ranks)", "ms": round(ms, 4),
                          "tflops": round(flops / ms / 1e9, 1)}))

    if what in ("moe", "all"):
        from tridist_b200.ops import (create_moe_a2a_intra_node_context, moe_combine_intra_node_op,
                                      moe_dispatch_intra_node_op)
        from tridist_b200.utils.testing import moe_inputs
        w = ProcessWorld(0, 1)
        E, H, T, topk = 64, 4096, 4096, 8
        h16 = torch.float16
        ctx = create_moe_a2a_intra_node_context(E, H, h16, T, topk, 0, 1, world=w)
        tokens, idx, wts = [x.cuda() for x in moe_inputs(0, T, H, E, topk, 0, h16)]
        out = torch.empty_like(tokens)
        ctx.out_buf, ctx.out = ctx.recv_buf, ctx.recv           # identity expert
        t_meta = timed(lambda: moe_dispatch_intra_node_op(tokens, idx, ctx, component="meta"), args.iters)
        t_disp = timed(lambda: moe_dispatch_intra_node_op(tokens, idx, ctx), args.iters)
        t_comb = timed(lambda: moe_combine_intra_node_op(ctx, idx, out, wts), args.iters)
        w.check(sync=True)
        rows_bytes = T * topk * H * 2
        print(json.dumps({"kernel": "moe_meta + moe_dispatch + moe_combine (1 rank)", "meta_ms": round(t_meta, 4),
                          "dispatch_ms": round(t_disp - t_meta, 4), "combine_ms": round(t_comb, 4),
                          "dispatch_gbs": round(2 * rows_bytes / ((t_disp - t_meta) * 1e6), 1),
                          "combine_gbs": round((rows_bytes + T * H * 2) / (t_comb * 1e6), 1),
                          "hbm_peak_gbs": peaks["hbm_gbs"], "peaks": peaks["source"]}))

    if what in ("swiglu", "all"):
        from tridist_b200.ops import swiglu
        rows, inter = 8192, 7168
        h = torch.randn(rows, 2 * inter, device="cuda").to(dt)
        o = torch.empty(rows, inter, dtype=dt, device="cuda")
        ms = timed(lambda: swiglu(h, o), args.iters)
        gbs = (h.numel() + o.numel()) * 2 / (ms * 1e6)
        print(json.dumps({"kernel": "swiglu_kernel", "ms": round(ms, 4), "gbs": round(gbs, 1),
                          "frac_of_copy_peak": round(gbs / peaks["hbm_gbs"], 3), "peaks": peaks["source"]}))


if __name__ == "__main__":
    main()
