"""Single-GPU probe of the hand-written tcgen05 GEMM against cuBLAS (torch.matmul).

The B200 counterpart of the reference's offline tile sweeps and native tile-GEMM probes
(bench/tune_gemm.py, bench/tune_gemm2.py, bench/dumma/p0b_tiled_gemm.cpp): there is no
runtime autotuner; this script sweeps the few knobs the kernel has —

  --bn {128,256}     output tile width
  --pair {0,1}       CTA pairs (2-CTA tcgen05 MMA on 256 x 256 tiles) on / off
  --ctas N           cap on the persistent grid
  --swiglu           SwiGLU epilogue (B holds [gate; up])

— checks the result against an fp32 reference and prints device-timed TFLOP/s for both
implementations. `--shapes M,N,K[;M,N,K...]`; `--iters`; `--once` runs a single launch of
each shape without timing (the form used under a profiler).

  python bench/probe_gemm.py --shapes "8192,6144,12288;8192,7168,8192" --dtype bf16
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="8192,6144,12288;8192,7168,8192;8192,8192,8192;4096,8192,3584")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--pair", type=int, default=1)
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--once", action="store_true")
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--probe", default="0", help="comma list of pipeline probes: 0 = the GEMM, 1 = tensor-pipe "
                    "ceiling (resident stages, no loads), 2 = operand-feed ceiling (loads, no MMAs)")
    ap.add_argument("--sustain-s", type=float, default=0.0, help="also time a back-to-back loop this long")
    args = ap.parse_args()
    os.environ["TRIDIST_CTA_PAIR"] = str(args.pair)

    import torch
    from tridist_b200.ops._gemm_common import gemm_nt
    from tridist_b200.utils.timing import flush_l2

    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    out_rows = []
    for shp in args.shapes.split(";"):
        M, N, K = [int(x) for x in shp.split(",")]
        torch.manual_seed(0)
        a = (torch.randn(M, K, device="cuda") * 0.05).to(dt)
        b = (torch.randn((2 * N if args.swiglu else N), K, device="cuda") * 0.05).to(dt)
        out = torch.empty(M, N, device="cuda", dtype=dt)
        kw = dict(bn=args.bn or None, swiglu=args.swiglu, max_ctas=args.ctas)
        gemm_nt(a, b, out=out, **kw)
        torch.cuda.synchronize()
        if args.once:
            continue
        # spot check against fp32 on a row/column sample (full fp32 products of these sizes are slow)
        rows = torch.randint(0, M, (64,), device="cuda")
        ref = a[rows].float() @ b.float().t()
        if args.swiglu:
            ref = torch.nn.functional.silu(ref[:, :N]) * ref[:, N:]
        err = (out[rows].float() - ref).abs().max().item()

        def timed(fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            ev = []
            for _ in range(args.iters):
                flush_l2()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                ev.append((e0, e1))
            torch.cuda.synchronize()
            ts = sorted(x.elapsed_time(y) for x, y in ev)
            return ts[len(ts) // 2]

        def sustained(fn):
            """Back-to-back launches for about --sustain-s seconds (no flush): the power-capped rate."""
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n = 0
            import time
            t_end = time.monotonic() + args.sustain_s
            e0.record()
            while time.monotonic() < t_end:
                for _ in range(20):
                    fn()
                n += 20
                torch.cuda.synchronize()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n

        flops = 2.0 * M * N * K * (2 if args.swiglu else 1)
        row = {"M": M, "N": N, "K": K, "dtype": args.dtype, "bn": args.bn or "auto", "pair": args.pair,
               "max_abs_err": err}
        for probe in [int(x) for x in args.probe.split(",")]:
            tag = {0: "ours", 1: "mma_only", 2: "feed_only"}[probe]
            fn = lambda: gemm_nt(a, b, out=out, probe=probe, **kw)  # noqa: E731
            t = timed(fn)
            row[tag + "_ms"] = round(t, 4)
            row[tag + "_tflops"] = round(flops / t / 1e9, 1)
            if args.sustain_s > 0:
                ts = sustained(fn)
                row[tag + "_sustained_tflops"] = round(flops / ts / 1e9, 1)
        t_ours = row.get("ours_ms")
        if not args.no_cublas and not args.swiglu:
            t_ref = timed(lambda: torch.matmul(a, b.t(), out=out))
            row["cublas_ms"] = round(t_ref, 4)
            row["cublas_tflops"] = round(flops / t_ref / 1e9, 1)
            if t_ours:
                row["ratio"] = round(t_ref / t_ours, 3)
            if args.sustain_s > 0:
                row["cublas_sustained_tflops"] = round(flops / sustained(lambda: torch.matmul(a, b.t(), out=out)) / 1e9, 1)
        print(json.dumps(row), flush=True)
        out_rows.append(row)


if __name__ == "__main__":
    main()
