"""Straggler-injection benchmark of the skew-aware all-gather + GEMM.

Counterpart of the reference's skew experiments (bench/s8_bench_skew.py, bench/l1_pred_bench.py,
bench/s20_bench_8card.py): one rank (the victim) is delayed on the HOST by delta microseconds
before it launches each round, which its peers see as a late shard. Three arms are compared on
the non-victim ranks:

  nopred   default source order (arrival order of an unskewed push)
  pred     order table from the sticky last-vote predictor, fed by the previous rounds'
           in-kernel arrival stamps
  oracle   the victim's shard always last

For every delta the script reports the mean device time of the op on the non-victim ranks,
the least-squares slope of time against delta per arm (1.0 = the delay is fully exposed,
0 = fully absorbed), and the predictor statistics. Injection is host-side sleep only.

Pass criteria, fixed before any run (in the spirit of the reference's pre-registered gates,
bench/l1_pred_aggregate.py C1-C5 and bench/s20_bench_8card.py G1-G3); the report carries one
verdict per criterion under "criteria":

  C1  no harm without skew: pred at delta = 0 is within 3 % (or 10 us) of nopred
  C2  the prediction helps: slope(pred) <= slope(nopred) - 0.03 when more than two ranks take
      part (with two ranks there is no order to choose, the criterion is recorded as "n/a")
  C3  the predictor finds the victim: degrade rate of the pred arm <= 0.25 over all rounds with skew
  C4  the oracle bounds the predictor: slope(pred) >= slope(oracle) - 0.10
  C5  correctness: the first and the last result of every arm match the fp32 reference on a row sample

  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/bench_skew.py \
      --m-per-rank 1024 --k 8192 --n-per-rank 3584 --deltas 0,100,200,400,800 --victim 3
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


def slope(xs, ys):
    n = len(xs)
    mx, my = sum(xs) / n, sum(ys) / n
    den = sum((x - mx) ** 2 for x in xs)
    return sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / den if den > 0 else 0.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m-per-rank", type=int, default=1024)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--n-per-rank", type=int, default=3584)
    ap.add_argument("--deltas", default="0,100,200,400,800")
    ap.add_argument("--victim", type=int, default=1)
    ap.add_argument("--rounds", type=int, default=24)
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    R = int(os.environ.get("WORLD_SIZE", "1"))
    assert R >= 2, "the skew benchmark needs at least two ranks"
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", rank=rank, world_size=R, device_id=torch.device("cuda", local_rank))

    from tridist_b200.ops import create_i1_context, i1_ag_tr_op, i1_table_write, observed_straggler
    from tridist_b200.parallel.predictor import StickyOrderPredictor
    from tridist_b200.parallel.runtime import init_runtime

    rt = init_runtime(rank, R)
    dt = torch.bfloat16
    m_pr, K, n_pr = args.m_per_rank, args.k, args.n_per_rank
    victim = args.victim % R
    a = (torch.randn(m_pr, K, device="cuda") * 0.05).to(dt)
    b = (torch.randn(n_pr, K, device="cuda") * 0.05).to(dt)
    c = torch.empty(m_pr * R, n_pr, dtype=dt, device="cuda")
    ictx = create_i1_context(m_pr * R, K, dt, dt, rank, R)
    deltas = [float(x) for x in args.deltas.split(",")]
    cfg = dict(vars(args))
    cfg.pop("out", None)                      # where the report goes is not part of the experiment
    report = {"config": cfg, "ranks": R, "arms": {}}
    rows = torch.arange(0, m_pr * R, max(1, (m_pr * R) // 64), device="cuda")[:64]
    a_all = [torch.empty_like(a) for _ in range(R)]
    dist.all_gather(a_all, a)
    ref_rows = torch.cat(a_all, 0)[rows].float() @ b.float().t()
    correct = True

    def pack(order):
        return sum(int(o) << (4 * i) for i, o in enumerate(order))

    for arm in ("nopred", "pred", "oracle"):
        per_delta = []
        pred = StickyOrderPredictor(rank, R)
        for delta in deltas:
            times = []
            for rnd in range(args.rounds):
                if arm == "nopred":
                    i1_table_write(ictx, rnd, 0, 0, pack(pred.rotation()), 1)
                elif arm == "oracle":
                    order = [rank] + [x for x in range(R) if x not in (rank, victim)] + ([victim] if victim != rank else [])
                    i1_table_write(ictx, rnd, 0, 1 if victim != rank else 0, pack(order), 1)
                else:
                    t = pred.table(k_eff=1)
                    i1_table_write(ictx, t["seq"], t["degraded"], t["mode"], t["order_packed"], t["k_eff"])
                rt.barrier_on_stream()
                torch.cuda.synchronize()
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                i1_ag_tr_op(a, b, c, ictx, stage_delay_us=delta if rank == victim else 0.0)
                e1.record()
                torch.cuda.synchronize()
                rt.check()
                if rnd in (0, args.rounds - 1):
                    correct &= bool((c[rows].float() - ref_rows).abs().max().item() < 2e-2)
                if arm == "pred":
                    pred.observe(observed_straggler(ictx) if delta > 0 else None)
                if rnd >= 4:                                    # first rounds warm the predictor
                    times.append(e0.elapsed_time(e1))
            mine = sum(times) / len(times)
            tt = torch.tensor([mine if rank != victim else 0.0, 1.0 if rank != victim else 0.0],
                              dtype=torch.float64, device="cuda")
            dist.all_reduce(tt)
            per_delta.append(round(float(tt[0] / tt[1]), 4))
        stats = pred.stats() if arm == "pred" else None
        report["arms"][arm] = {"mean_ms_non_victim": dict(zip([str(d) for d in deltas], per_delta)),
                               "slope_ms_per_ms": round(slope([d / 1e3 for d in deltas], per_delta), 3),
                               "predictor": stats}
        if rank == 0:
            print(arm, json.dumps(report["arms"][arm]), flush=True)
    ok_all = torch.tensor([1.0 if correct else 0.0], device="cuda")
    dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
    arms = report["arms"]
    z = str(deltas[0])
    t0_pred, t0_no = arms["pred"]["mean_ms_non_victim"][z], arms["nopred"]["mean_ms_non_victim"][z]
    s_pred, s_no, s_or = (arms[k]["slope_ms_per_ms"] for k in ("pred", "nopred", "oracle"))
    report["criteria"] = {
        "C1_no_harm_at_zero_delay": bool(deltas[0] != 0 or t0_pred <= max(t0_no * 1.03, t0_no + 0.010)),
        "C2_prediction_helps": (bool(s_pred <= s_no - 0.03) if R > 2 else "n/a"),
        "C3_victim_found": bool((arms["pred"]["predictor"] or {}).get("degrade_rate", 1.0) <= 0.25),
        "C4_oracle_bounds_predictor": bool(s_pred >= s_or - 0.10),
        "C5_results_correct": bool(ok_all.item() > 0),
    }
    if rank == 0:
        print("criteria", json.dumps(report["criteria"]), flush=True)
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as fh:
            json.dump(report, fh, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
