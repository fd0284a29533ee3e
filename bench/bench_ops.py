"""Per-operator benchmark with decomposition, in the style of the reference's op benches
(bench/s4_bench.py, s6_bench_gemm_ar.py, s7_bench_moe_a2a.py, s9_bench_8card.py): for every
operator and shape it times the fused call, its GEMM-only / communication-free component,
and the cuBLAS + NCCL composition together with its two parts, after checking the result.

  python bench/bench_ops.py --ops ag,rs,ar,moe [--iters 20] [--out bench/results/ops.json]
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/bench_ops.py ...

Every number is device-timed (event pairs enqueued back to back, one synchronisation at
the end), p50 over iterations of the max over ranks, with an L2 flush and a device-side
barrier of all ranks before each timed call. Cells are written to the JSON file as they
finish and cells already present are skipped (resumable, like the reference's sweeps).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="ag,rs,ar,moe")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    ap.add_argument("--small", action="store_true", help="reduced shapes (quick functional pass)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    R = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if R > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=R, device_id=torch.device("cuda", local_rank))

    from bench import baselines
    from tridist_b200.ops import (ag_gemm_intra_node_op, create_ag_gemm_intra_node_context,
                                  create_gemm_ar_intra_node_context, create_gemm_rs_intra_node_context,
                                  create_moe_a2a_intra_node_context, gemm_ar_intra_node_op,
                                  gemm_rs_intra_node_op, moe_combine_intra_node_op, moe_dispatch_intra_node_op)
    from tridist_b200.ops._gemm_common import gemm_nt
    from tridist_b200.parallel.runtime import init_runtime
    from tridist_b200.utils import roofline
    from tridist_b200.utils.testing import moe_inputs
    from tridist_b200.utils.timing import time_op

    rt = init_runtime(rank, R)
    results = {}
    if args.out and os.path.exists(args.out):
        with open(args.out) as fh:
            results = json.load(fh)

    def t(fn):
        return round(time_op(fn, iters=args.iters, warmup=3, flush=True, barrier=rt.barrier_on_stream)["p50"], 4)

    def prof_of(fn):
        """One more call with the stall accounting read back (only with TRIDIST_PROF=1)."""
        from tridist_b200.ops._gemm_common import prof_buffer, read_prof
        if prof_buffer() is None:
            return None
        for _ in range(3):                       # keep the GPU busy: the accounted call runs at load clocks
            rt.barrier_on_stream()
            fn()
        prof_buffer().zero_()
        rt.barrier_on_stream()
        fn()
        torch.cuda.synchronize()
        return read_prof()

    def emit(name, cell):
        results[name] = cell
        if rank == 0:
            print(name, json.dumps(cell), flush=True)
            if args.out:
                os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
                with open(args.out, "w") as fh:
                    json.dump(results, fh, indent=1)

    def randn(shape, seed, scale, dt):
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        return (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(dt)

    ops = args.ops.split(",")
    dt = torch.float16
    sc = 8 if args.small else 1

    if "ag" in ops:
        for (M, K, N) in [(8192 // sc, 12288 // sc, 49152 // sc), (8192 // sc, 8192 // sc, 57344 // sc)]:
            name = f"ag_gemm_M{M}_K{K}_N{N}_R{R}"
            if name in results:
                continue
            m_pr, n_loc = M // R, N // R
            a = randn((m_pr, K), 1 + rank, 1 / math.sqrt(K), dt)
            b = randn((n_loc, K), 100 + rank, 1 / math.sqrt(K), dt)
            c = torch.empty((M, n_loc), dtype=dt, device="cuda")
            ctx = create_ag_gemm_intra_node_context(M, K, dt, dt, rank, R, M_PER_CHUNK=m_pr)
            base = baselines.AGGemmBaseline(m_pr, K, n_loc, R, dt)
            ag_gemm_intra_node_op(a, b, c, ctx)
            err = (c.float() - base(a, b).float()).abs().max().item()
            cell = {"fused": t(lambda: ag_gemm_intra_node_op(a, b, c, ctx)),
                    "fused_gemm_only": t(lambda: ag_gemm_intra_node_op(a, b, c, ctx, skip_comm=True)),
                    "cublas_nccl": t(lambda: base(a, b)),
                    "cublas_only": t(lambda: torch.matmul(base.full, b.t(), out=base.c)),
                    "roofline": round(roofline.ag_gemm_roof(M, K, n_loc, R)["ms"], 4), "err": err}
            if R > 1:
                cell["nccl_only"] = t(lambda: dist.all_gather_into_tensor(base.full, a))
                cell["fused_push_only"] = t(lambda: ag_gemm_intra_node_op(a, b, c, ctx, comm_only=True))
            pr = prof_of(lambda: ag_gemm_intra_node_op(a, b, c, ctx))
            if pr:
                cell["prof_us"] = pr
                cell["prof_gemm_only_us"] = prof_of(lambda: ag_gemm_intra_node_op(a, b, c, ctx, skip_comm=True))
            emit(name, cell)
            rt.check(sync=True)

    if "rs" in ops:
        for (M, K, N) in [(8192 // sc, 49152 // sc, 12288 // sc), (8192 // sc, 28672 // sc, 8192 // sc)]:
            name = f"gemm_rs_M{M}_K{K}_N{N}_R{R}"
            if name in results:
                continue
            kl = K // R
            a = randn((M, kl), 2 + rank, 1 / math.sqrt(K), dt)
            b = randn((N, kl), 200 + rank, 1 / math.sqrt(K), dt)
            out = torch.empty((M // R, N), dtype=dt, device="cuda")
            full = torch.empty((M, N), dtype=dt, device="cuda")
            ctx = create_gemm_rs_intra_node_context(M, N, dt, rank, R)
            base = baselines.GemmRSBaseline(M, N, R, dt)
            gemm_rs_intra_node_op(a, b, dt, rank, R, ctx, out=out)
            err = (out.float() - base(a, b).float()).abs().max().item()
            cell = {"fused": t(lambda: gemm_rs_intra_node_op(a, b, dt, rank, R, ctx, out=out)),
                    "fused_gemm_only": t(lambda: gemm_nt(a, b, out=full)),
                    "cublas_nccl": t(lambda: base(a, b)),
                    "cublas_only": t(lambda: torch.matmul(a, b.t(), out=base.partial)),
                    "roofline": round(roofline.gemm_rs_roof(M, N, kl, R)["ms"], 4), "err": err}
            if R > 1:
                cell["nccl_only"] = t(lambda: dist.reduce_scatter_tensor(base.out, base.partial))
            pr = prof_of(lambda: gemm_rs_intra_node_op(a, b, dt, rank, R, ctx, out=out))
            if pr:
                cell["prof_us"] = pr
            emit(name, cell)
            rt.check(sync=True)

    if "ar" in ops:
        K, N = 28672 // sc, 8192 // sc
        for M in [128, 1024, 4096 // sc if not args.small else 512]:
            name = f"gemm_ar_M{M}_K{K}_N{N}_R{R}"
            if name in results:
                continue
            kl = K // R
            a = randn((M, kl), 3 + rank, 1 / math.sqrt(K), dt)
            b = randn((N, kl), 300 + rank, 1 / math.sqrt(K), dt)
            c = torch.empty((M, N), dtype=dt, device="cuda")
            ctx = create_gemm_ar_intra_node_context(M, N, dt, dt, rank, R, M_PER_CHUNK=64, nvls=R > 1)
            base = baselines.GemmARBaseline(M, N, R, dt)
            cell = {}
            ref = base(a, b).float()
            for mode in (["one_shot", "two_shot"] if R > 1 else ["auto"]):
                ctx.mode = mode
                gemm_ar_intra_node_op(a, b, c, ctx)
                cell[f"err_{mode}"] = (c.float() - ref).abs().max().item()
                cell[f"fused_{mode}"] = t(lambda: gemm_ar_intra_node_op(a, b, c, ctx))
            if R > 1:
                ctx.mode = "two_shot"
                cs = ctx.symm_output(M)
                cell["fused_two_shot_symm_c"] = t(lambda: gemm_ar_intra_node_op(a, b, ctx.symm_output(M), ctx))
                del cs
                if ctx.mc is not None:
                    # two-shot with the reduction and the replication done by the switch
                    ctx.mode = "nvls"
                    gemm_ar_intra_node_op(a, b, c, ctx)
                    cell["err_nvls"] = (c.float() - ref).abs().max().item()
                    cell["fused_nvls"] = t(lambda: gemm_ar_intra_node_op(a, b, c, ctx))
                    cell["fused_nvls_symm_c"] = t(lambda: gemm_ar_intra_node_op(a, b, ctx.symm_output(M), ctx))
                else:
                    cell["nvls"] = "unavailable: " + str(getattr(rt, "multicast_unavailable", "off"))
                cell["nccl_only"] = t(lambda: dist.all_reduce(base.c))
            for mode in ((["two_shot"] + (["nvls"] if ctx.mc is not None else [])) if R > 1 else [ctx.mode]):
                ctx.mode = mode
                pr = prof_of(lambda: gemm_ar_intra_node_op(a, b, ctx.symm_output(M) if R > 1 else c, ctx))
                if pr:
                    cell["prof_us_" + mode] = pr
            if R > 1 and R & (R - 1) == 0 and M >= 256:
                # the recursive-doubling transport of the "rd" entry points: panel GEMMs + XOR-partner exchange
                from tridist_b200.ops import (create_gemm_ar_rd_context, finalize_gemm_ar_rd_context,
                                              gemm_ar_rd_op)
                rd = create_gemm_ar_rd_context(M, N, dt, dt, rank, R, transport="rd")
                gemm_ar_rd_op(a, b, c, rd)
                cell["err_rd"] = (c.float() - ref).abs().max().item()
                cell["fused_rd"] = t(lambda: gemm_ar_rd_op(a, b, c, rd))
                cell["rd_panels"] = -(-M // rd.rd.chunk_rows)
                finalize_gemm_ar_rd_context(rd)
            cell["fused_gemm_only"] = t(lambda: gemm_ar_intra_node_op(a, b, c, ctx, component="gemm"))
            cell["cublas_nccl"] = t(lambda: base(a, b))
            cell["cublas_only"] = t(lambda: torch.matmul(a, b.t(), out=base.c))
            cell["roofline_two_shot"] = round(roofline.gemm_ar_roof(M, N, kl, R, True)["ms"], 4)
            cell["roofline_one_shot"] = round(roofline.gemm_ar_roof(M, N, kl, R, False)["ms"], 4)
            emit(name, cell)
            rt.check(sync=True)

    if "moe" in ops:
        E, H, T, topk = 64, 4096 // sc, 4096 // sc, 8
        for zipf in (0.0, 1.2):
            name = f"moe_a2a_T{T}_H{H}_E{E}_topk{topk}_zipf{zipf}_R{R}"
            if name in results:
                continue
            tokens, idx, wts = [x.cuda() for x in moe_inputs(rank, T, H, E, topk, 0, dt, zipf)]
            out = torch.empty_like(tokens)
            ctx = create_moe_a2a_intra_node_context(E, H, dt, T, topk, rank, R)
            base = baselines.MoEBaseline(idx, E, H, R, dt)
            n = int(moe_dispatch_intra_node_op(tokens, idx, ctx).item())
            ctx.out[:n].copy_(ctx.recv[:n])
            moe_combine_intra_node_op(ctx, idx, out, wts)
            err = (out.float() - tokens.float()).abs().max().item()

            def round_trip():
                moe_dispatch_intra_node_op(tokens, idx, ctx)
                moe_combine_intra_node_op(ctx, idx, out, wts)

            cell = {"round": t(round_trip),
                    "dispatch": t(lambda: moe_dispatch_intra_node_op(tokens, idx, ctx)),
                    "meta": t(lambda: moe_dispatch_intra_node_op(tokens, idx, ctx, component="meta")),
                    "nccl_a2a_x2": t(base), "err": err, "recv_rows": n}
            # combine alone needs a dispatch of the same round before it; time the pair and subtract
            cell["combine"] = round(cell["round"] - cell["dispatch"], 4)
            emit(name, cell)
            rt.check(sync=True)

    torch.cuda.synchronize()
    if R > 1:
        dist.barrier()
        rt.release_multicast()      # no rank leaves while bound to a multicast object
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
