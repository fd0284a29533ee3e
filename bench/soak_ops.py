"""Numerical soak of the fused operators: many rounds on ONE context per operator, fresh seeded
data every round, every result checked against an fp32 reference built from all ranks' seeds.

Counterpart of the reference's soak rig (tests/dbg_rsar_soak.py): it exists to catch what a
three-round acceptance test cannot, such as a workspace generation reused too early, a ticket
that is one round stale, or a rare torn tile. On a mismatch the round, the operator, the worst
element and the rows that differ are reported (rows localise a bad tile or a bad source shard)
and the soak goes on, so that the failure RATE is known at the end.

  python bench/soak_ops.py --rounds 200                                  one GPU (R = 1 degenerate paths)
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/soak_ops.py --rounds 600
  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/soak_ops.py --device cpu \
      --rounds 20 --small                                                gloo oracle backend
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def _report(problems, op, rnd, got, ref, tol):
    diff = (got.float() - ref.float()).abs()
    worst = diff.max().item()
    if worst < tol:
        return worst
    bad_rows = (diff.max(dim=1).values >= tol).nonzero().flatten().tolist()
    problems.append({"op": op, "round": rnd, "max_abs_err": worst, "bad_rows": bad_rows[:16],
                     "n_bad_rows": len(bad_rows)})
    return worst


def soak(rank: int, R: int, world, rounds: int, small: bool, dtype, tol: float, ops=("ag", "rs", "ar", "moe")):
    """Runs the soak on an initialised world; returns (per-op worst error, list of problems)."""
    from tridist_b200.ops import (ag_gemm_intra_node_op, create_ag_gemm_intra_node_context,
                                  create_gemm_ar_intra_node_context, create_gemm_rs_intra_node_context,
                                  create_moe_a2a_intra_node_context, finalize_ag_gemm_context,
                                  finalize_gemm_ar_context, finalize_gemm_rs_context, finalize_moe_a2a_context,
                                  gemm_ar_intra_node_op, gemm_rs_intra_node, moe_combine_intra_node_op,
                                  moe_dispatch_intra_node_op)
    from tridist_b200.utils.testing import ag_inputs, fake_expert, ks_inputs, moe_inputs
    dev = "cpu" if world.kind == "cpu" else "cuda"
    sync = (lambda: None) if dev == "cpu" else torch.cuda.synchronize
    worst = {}
    problems = []
    if "ag" in ops:
        m_pr, K, n_pr = (128, 256, 128) if small else (1024, 4096, 2048)
        ctx = create_ag_gemm_intra_node_context(m_pr * R, K, dtype, dtype, rank, R, M_PER_CHUNK=m_pr, world=world)
        c = torch.empty(m_pr * R, n_pr, dtype=dtype, device=dev)
        for rnd in range(rounds):
            a_all, b = ag_inputs(rank, R, m_pr, K, n_pr, rnd, dtype, device=dev)
            ag_gemm_intra_node_op(a_all[rank].to(dev), b.to(dev), c, ctx)
            sync()
            world.check()
            ref = torch.cat(a_all, 0).to(dev).float() @ b.to(dev).float().t()
            worst["ag"] = max(worst.get("ag", 0.0), _report(problems, "ag_gemm", rnd, c, ref, tol))
        finalize_ag_gemm_context(ctx)
    if "rs" in ops or "ar" in ops:
        M, N, kl = (256, 128, 64) if small else (2048, 2048, 1024)
        rs = create_gemm_rs_intra_node_context(M, N, dtype, rank, R, world=world) if "rs" in ops else None
        ar = create_gemm_ar_intra_node_context(M, N, dtype, dtype, rank, R, M_PER_CHUNK=64, world=world) \
            if "ar" in ops else None
        c = torch.empty(M, N, dtype=dtype, device=dev)
        m_pr = M // R
        for rnd in range(rounds):
            a_all, b_all = ks_inputs(R, M, N, kl, rnd, dtype, device=dev)
            ref = sum(a_all[s].to(dev).float() @ b_all[s].to(dev).float().t() for s in range(R))
            a, b = a_all[rank].to(dev), b_all[rank].to(dev)
            if rs is not None:
                out = gemm_rs_intra_node(a, b, rs)
                sync()
                world.check()
                worst["rs"] = max(worst.get("rs", 0.0),
                                  _report(problems, "gemm_rs", rnd, out, ref[rank * m_pr:(rank + 1) * m_pr], tol))
            if ar is not None:
                gemm_ar_intra_node_op(a, b, c, ar)
                sync()
                world.check()
                worst["ar"] = max(worst.get("ar", 0.0), _report(problems, "gemm_ar", rnd, c, ref, tol))
        if rs is not None:
            finalize_gemm_rs_context(rs)
        if ar is not None:
            finalize_gemm_ar_context(ar)
    if "moe" in ops:
        E, H, topk, T = (4 * R, 64, 2, 32) if small else (8 * R, 1024, 4, 512)
        ctx = create_moe_a2a_intra_node_context(E, H, dtype, T, topk, rank, R, world=world)
        out = torch.empty(T, H, dtype=dtype, device=dev)
        for rnd in range(rounds):
            tokens, idx, wts = [x.to(dev) for x in moe_inputs(rank, T, H, E, topk, rnd, dtype,
                                                              1.2 if rnd % 3 == 2 else 0.0)]
            n = int(moe_dispatch_intra_node_op(tokens, idx, ctx).item())
            world.check()
            ctx.out[:n] = fake_expert(ctx.recv[:n])
            moe_combine_intra_node_op(ctx, idx, out, wts)
            sync()
            world.check()
            sc = ctx.scatter_idx[:T].long()
            ref = (wts.unsqueeze(-1) * (tokens.float().unsqueeze(1) * 2 + (sc % 5).float().unsqueeze(-1))).sum(1)
            worst["moe"] = max(worst.get("moe", 0.0), _report(problems, "moe_a2a", rnd, out, ref, 3 * tol))
        finalize_moe_a2a_context(ctx)
    return worst, problems


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rounds", type=int, default=100)
    ap.add_argument("--ops", default="ag,rs,ar,moe")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--small", action="store_true", help="tiny shapes (CPU backend, quick functional pass)")
    ap.add_argument("--tol", type=float, default=1e-2)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    R = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if args.device == "cuda":
        torch.cuda.set_device(local_rank)
    if R > 1:
        if args.device == "cuda":
            dist.init_process_group("nccl", rank=rank, world_size=R, device_id=torch.device("cuda", local_rank))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=R)
    from tridist_b200.parallel.runtime import init_runtime
    world = init_runtime(rank, R, device=args.device)
    dtype = torch.float32 if args.device == "cpu" else torch.float16
    worst, problems = soak(rank, R, world, args.rounds, args.small, dtype,
                           1e-4 if args.device == "cpu" else args.tol, tuple(args.ops.split(",")))
    summary = {"rank": rank, "ranks": R, "rounds": args.rounds, "device": args.device,
               "worst_abs_err": {k: round(v, 6) for k, v in worst.items()},
               "failed_rounds": len(problems), "problems": problems[:20]}
    if R > 1:
        all_s = [None] * R
        dist.all_gather_object(all_s, summary)
    else:
        all_s = [summary]
    if rank == 0:
        total = {"ranks": R, "rounds": args.rounds, "device": args.device,
                 "failed_rounds": sum(s["failed_rounds"] for s in all_s),
                 "worst_abs_err": {k: max(s["worst_abs_err"].get(k, 0.0) for s in all_s)
                                   for k in all_s[0]["worst_abs_err"]},
                 "per_rank": all_s}
        print(json.dumps({k: v for k, v in total.items() if k != "per_rank"}))
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            with open(args.out, "w") as fh:
                json.dump(total, fh, indent=1)
    world.release_multicast()
    if R > 1:
        dist.barrier()
        dist.destroy_process_group()
    sys.exit(1 if problems else 0)


if __name__ == "__main__":
    main()
