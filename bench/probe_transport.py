"""Transport probes over the symmetric heap (two or more GPUs).

The B200 counterpart of the reference's transport micro-benchmarks (bench/s4_transport_probe.py,
bench/s7_peer_load_probe.py, bench/s5_signal_probe.py, bench/s9_probe_8pe.py): what the fabric
gives to the mechanisms the fused operators are built from.

  peer_copy        device-to-peer copy of a large buffer (copy kernel / engine chosen by torch)
  push_kernel      the library's own in-kernel all-gather push (bulk copies driven by one thread
                   per pushing CTA), for several numbers of pushing CTAs
  signal_latency   set a flag word in the peer's heap, the peer waits for it and answers
                   (half the round trip of the ping-pong is reported)
  barrier          the device-side ticket barrier of all ranks
  heap_capacity    allocate / free symmetric buffers of growing size up to --max-gb

  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/probe_transport.py
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=256)
    ap.add_argument("--max-gb", type=float, default=8.0)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    R = int(os.environ.get("WORLD_SIZE", "1"))
    assert R >= 2
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", rank=rank, world_size=R, device_id=torch.device("cuda", local_rank))
    from tridist_b200.ops import ag_gemm_intra_node_op, create_ag_gemm_intra_node_context, finalize_ag_gemm_context
    from tridist_b200.parallel.runtime import init_runtime
    from tridist_b200.parallel.symm_host import SymmHost
    from tridist_b200.utils.timing import time_op
    rt = init_runtime(rank, R)
    host = SymmHost(rt)
    out = {}
    peer = (rank + 1) % R

    # ---- peer copy -----------------------------------------------------------------
    nbytes = args.mb << 20
    buf = host.malloc(nbytes)
    src = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    r = time_op(lambda: host.putmem(buf, 0, src, peer), iters=args.iters, warmup=2, flush=False,
                barrier=rt.barrier_on_stream)
    out["peer_copy_gbs"] = round(nbytes / (r["p50"] * 1e6), 1)
    host.free(buf)

    # ---- in-kernel push ----------------------------------------------------------------
    m_pr, K = 2048, 8192
    a = torch.empty(m_pr, K, dtype=torch.bfloat16, device="cuda").normal_()
    b = torch.empty(256, K, dtype=torch.bfloat16, device="cuda").normal_()
    c = torch.empty(m_pr * R, 256, dtype=torch.bfloat16, device="cuda")
    out["push_kernel"] = {}
    for ctas in (8, 16, 32, 64, 0):
        os.environ["TRIDIST_PUSH_CTAS"] = str(ctas)
        ctx = create_ag_gemm_intra_node_context(m_pr * R, K, torch.bfloat16, torch.bfloat16, rank, R, M_PER_CHUNK=m_pr)
        r = time_op(lambda: ag_gemm_intra_node_op(a, b, c, ctx, comm_only=True), iters=args.iters, warmup=2,
                    flush=False, barrier=rt.barrier_on_stream)
        sent = (R - 1) * m_pr * K * 2
        out["push_kernel"][str(ctas or "all")] = {"ms": round(r["p50"], 4), "egress_gbs": round(sent / (r["p50"] * 1e6), 1)}
        torch.cuda.synchronize()
        finalize_ag_gemm_context(ctx)
    os.environ.pop("TRIDIST_PUSH_CTAS", None)

    # ---- signal latency (ranks 0 and 1 play ping-pong, the others idle) --------------------
    flags = host.malloc(256)
    rounds = 200
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if rank in (0, 1):
        other = 1 - rank
        for i in range(1, rounds + 1):
            if rank == 0:
                host.set_signal(flags, 0, i, other)
                host.wait_signal(flags, 1, i)
            else:
                host.wait_signal(flags, 0, i)
                host.set_signal(flags, 1, i, other)
    e1.record()
    torch.cuda.synchronize()
    rt.check()
    out["signal_one_way_us"] = round(e0.elapsed_time(e1) * 1e3 / rounds / 2, 2)   # includes two kernel launches per leg
    host.free(flags)

    # ---- barrier ---------------------------------------------------------------------------
    r = time_op(rt.barrier_on_stream, iters=50, warmup=5, flush=False)
    out["barrier_us"] = round(r["p50"] * 1e3, 2)

    # ---- heap capacity ladder ---------------------------------------------------------------
    ladder, gb = [], 0.5
    while gb <= args.max_gb:
        try:
            bfr = host.malloc(int(gb * (1 << 30)))
            host.free(bfr)
            ladder.append(gb)
        except RuntimeError:
            break
        gb *= 2
    out["heap_capacity_ok_gb"] = ladder
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
