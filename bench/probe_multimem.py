"""Transport probe of the NVSwitch multicast path (multimem.ld_reduce + multimem.st), in the
spirit of the reference's transport probes (bench/s4_transport_probe.py): how does the
switch-reduced all-reduce throughput of one rank depend on the number of threads, on the
16-byte pieces each thread keeps in flight, on the ordering qualifier (.relaxed.sys / .weak)
and on where the result goes (replicated through the switch / local store)?

Every rank reduces its own 1/R of the buffer, all ranks at once, as a two-shot all-reduce
does. Device-timed, max over ranks, median of the repetitions.

  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/probe_multimem.py \
      [--mb 64] [--out bench/results/multimem_2xB200.json]
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=64, help="buffer size (all ranks together reduce this much)")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    R = int(os.environ.get("WORLD_SIZE", "1"))
    if R < 2:
        print(json.dumps({"unavailable": "needs at least two ranks"}))
        return
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", rank=rank, world_size=R, device_id=torch.device("cuda", local_rank))
    from tridist_b200.parallel.runtime import init_runtime, native
    from tridist_b200.utils.timing import max_over_ranks
    rt = init_runtime(rank, R)
    nbytes = args.mb << 20
    buf = rt.alloc_multicast(2 * nbytes)
    if buf is None:
        if rank == 0:
            print(json.dumps({"unavailable": str(getattr(rt, "multicast_unavailable", "no multicast"))}))
        dist.destroy_process_group()
        return
    C = native()
    src = buf.tensor(torch.bfloat16, (nbytes // 2,), 0)
    src.fill_(float(rank + 1))
    local = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    pieces = nbytes // 16
    begin, end = rank * pieces // R, (rank + 1) * pieces // R
    rows = []
    rt.host_barrier()
    for blocks, threads in ((32, 128), (148, 128), (148, 256), (148, 512), (148, 1024), (296, 1024), (32, 1024)):
        for unroll in (1, 4, 8):
            for weak, local_store in ((False, False), (True, False), (False, True)):
                def launch():
                    C.multimem_probe(buf.mc_ptr, buf.mc_ptr + nbytes, local.data_ptr(), begin, end, blocks,
                                     threads, unroll, weak, local_store)
                times = []
                for rep in range(args.reps + 1):
                    rt.barrier_on_stream()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    launch()
                    e1.record()
                    torch.cuda.synchronize()
                    if rep:
                        times.append(e0.elapsed_time(e1))
                ms = max_over_ranks([statistics.median(times)])[0]
                rows.append({"blocks": blocks, "threads": threads, "in_flight_per_thread": unroll,
                             "order": "weak" if weak else "relaxed.sys",
                             "store": "local" if local_store else "multimem.st",
                             "ms": round(ms, 4),
                             "reduced_gbs_per_rank": round((end - begin) * 16 / ms / 1e6, 1)})
    # the replicated result of the last multimem.st pass: sum over ranks of (rank + 1)
    res = buf.tensor(torch.bfloat16, (nbytes // 2,), nbytes)
    torch.cuda.synchronize()
    rt.host_barrier()
    ok = bool((res.float() == R * (R + 1) / 2).all().item())
    oks = max_over_ranks([0.0 if ok else 1.0])[0] == 0.0
    if rank == 0:
        out = {"ranks": R, "mb": args.mb, "result_correct_on_all_ranks": oks, "rows": rows}
        for r in rows:
            print(json.dumps(r))
        print(json.dumps({"result_correct_on_all_ranks": oks}))
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            with open(args.out, "w") as fh:
                json.dump(out, fh, indent=1)
    rt.release_multicast()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
