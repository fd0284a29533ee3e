"""Skew-aware all-gather + GEMM: table-driven tile order, arrival observer, verify + repair.

Public entry points of the reference's "I1" layer
(triton_dist/kernels/dcu/ag_tr_pred.py:599-1131) on top of the fused AG+GEMM kernel:

* ``create_i1_context`` / ``finalize_i1_context``
* ``i1_table_write(ictx, seq, deg, mode, order_packed, k_eff)``: publishes this forward's
  table ``[seq, degraded, mode, k_eff, order[R], budget[R]]`` (int32 words) to device memory
* ``i1_ag_tr_op(a, b, c, ictx, stage_delay_us=0.0, with_observer=True)``: one AG+GEMM whose
  consumer reads the table on the device: ``mode == 1`` walks the source segments in the
  table's order, source-major (predicted-early sources first, predicted straggler last);
  ``mode == 0`` walks ``k_eff`` row bands band-major (band 0 of every source, then band 1, ...)
  in the table's order; ``degraded == 1`` ignores the order and walks the default rotation
  band-major; ``budget[s]`` is the number of polls of source s's ticket between two looks at
  the abort word and the clock
* ``i1_observer_read(ictx)``: ``[round, order by first-seen arrival..., arrival offsets in ns...]``
* ``calibrate_sleep_cycles_per_us``

Differences from the reference, by design: the tile order is read by the kernel from
device memory (no re-specialisation), the observer is not a separate polling kernel
but a ``globaltimer`` stamp taken by the consumer's TMA warp when it first finds a
source's ticket raised, and straggler injection is a host-side sleep before the
launch (the reference documents device-side sleeps as unsafe,
bench/l1_pred_bench.py:32-36). Verification (``TRIDIST_VERIFY=1``; off by default —
the tear it guarded against in the reference is specific to that platform,
docs/AG_TEAR_FIX_20261014.md:12-22) recomputes a few elements per tile and re-runs
flagged tiles through the same GEMM mainloop with a list-driven scheduler.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..parallel.runtime import CpuWorld, native
from ..utils.config import env_flag, env_float, env_int
from ._gemm_common import OP_AG, SCHED_LIST, base_desc, choose_bn
from .all_gather_gemm import ag_gemm_intra_node_op
from .gemm_ag_tr import create_gemm_ag_tr_context, finalize_gemm_ag_tr_context

TABLE_HEADER_WORDS = 4
INT64_MAX = (1 << 63) - 1


@dataclass
class I1PredContext:
    ag: object
    budget: int
    table: torch.Tensor                 # device int32 [4 + 2R]
    table_host: torch.Tensor            # pinned staging of the same words
    mode: int = 0
    seq: int = 0
    verify_hits: int = 0
    last_round: int = 0
    _bad: Optional[torch.Tensor] = field(default=None, repr=False)

    @property
    def order_ptr(self) -> int:
        return self.table.data_ptr() + TABLE_HEADER_WORDS * 4


def create_i1_context(max_M, K, input_dtype, output_dtype, rank, num_ranks, mpi=None, comm=None,
                      chunk_rows=0, comm_lanes=2, wait_mode=None, budget=128, world=None):
    ag = create_gemm_ag_tr_context(max_M=max_M, K=K, input_dtype=input_dtype, output_dtype=output_dtype,
                                   rank=rank, num_ranks=num_ranks, mpi=mpi, comm=comm, chunk_rows=chunk_rows,
                                   comm_lanes=comm_lanes, wait_mode=wait_mode, world=world)
    ag.observe = True
    words = TABLE_HEADER_WORDS + 2 * num_ranks
    dev = "cpu" if isinstance(ag.world, CpuWorld) else "cuda"
    table = torch.zeros(words, dtype=torch.int32, device=dev)
    host = torch.zeros(words, dtype=torch.int32)
    if dev == "cuda":
        host = host.pin_memory()
    ictx = I1PredContext(ag=ag, budget=budget, table=table, table_host=host)
    i1_table_write(ictx, 0, 0, 0, sum(((rank + i) % num_ranks) << (4 * i) for i in range(num_ranks)), 1)
    return ictx


def finalize_i1_context(ictx) -> None:
    finalize_gemm_ag_tr_context(ictx.ag)


def i1_table_write(ictx, seq, deg, mode, order_packed, k_eff) -> None:
    """Stream-ordered update of the table; ``order_packed`` holds 4 bits per slot."""
    R = ictx.ag.num_ranks
    order = [(int(order_packed) >> (4 * i)) & 0xF for i in range(R)]
    assert sorted(order) == list(range(R)), "order must be a permutation of the ranks"
    h = ictx.table_host
    h[0], h[1], h[2], h[3] = int(seq), int(deg), int(mode), int(k_eff)
    for i, r in enumerate(order):
        h[TABLE_HEADER_WORDS + i] = r
        h[TABLE_HEADER_WORDS + R + i] = ictx.budget
    ictx.table.copy_(h, non_blocking=True)
    ictx.mode, ictx.seq = int(mode), int(seq)


def i1_table_peek(ictx) -> List[int]:
    """Host copy of the device table (the reference's peek kernel, ag_tr_pred.py:273)."""
    return ictx.table.cpu().tolist()


def _verify_and_repair(a, b, c, ictx) -> int:
    ag = ictx.ag
    C = native()
    R = ag.num_ranks
    m_pr, K = a.shape
    M, N = m_pr * R, b.shape[0]
    bn = choose_bn(M, N)
    n_tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
    if ictx._bad is None or ictx._bad.numel() < n_tiles:
        ictx._bad = torch.zeros(n_tiles, dtype=torch.int32, device="cuda")
    bad = ictx._bad[:n_tiles]
    bad.zero_()
    if R > 1:
        full = ag.workspace(ag.flag_round & 1, M)
        full[ag.rank * m_pr:(ag.rank + 1) * m_pr].copy_(a)       # own rows are not pushed to self
    else:
        full = a
    C.spot_verify(full.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, full.stride(0), b.stride(0), c.stride(0),
                  a.dtype == torch.bfloat16, env_int("TRIDIST_VERIFY_SPOTS", 4),
                  env_float("TRIDIST_VERIFY_TOL", 2e-2), bad.data_ptr(), bn)
    ids = torch.nonzero(bad).flatten().to(torch.int32)            # host sync: the reference reads flags too
    if ids.numel() == 0:
        return 0
    d = base_desc(ag.world, 0, 1, full, b, c.data_ptr(), c.stride(0), M, N, K, bn, OP_AG)
    d["sched"] = SCHED_LIST
    d["tile_list"] = ids.data_ptr()
    d["list_len"] = int(ids.numel())
    pid = C.gemm_plan_create(d)
    C.gemm_plan_launch(pid, 1, 0, 0, 1)
    torch.cuda.current_stream().synchronize()
    C.gemm_plan_destroy(pid)
    return int(ids.numel())


def i1_ag_tr_op(a, b, c, ictx, stage_delay_us: float = 0.0, with_observer: bool = True):
    """AG+GEMM with the table-driven consumer. ``stage_delay_us`` > 0 delays this rank's
    launch on the host, which the peers see as pure arrival skew of this rank's shard."""
    ag = ictx.ag
    if stage_delay_us > 0:
        time.sleep(stage_delay_us * 1e-6)
    ag.observe = bool(with_observer)
    if isinstance(ag.world, CpuWorld):
        return ag_gemm_intra_node_op(a, b, c, ag)
    # the kernel reads the whole table: degraded / mode / k_eff in front of order[], budget[] behind
    table = ictx.table[TABLE_HEADER_WORDS:TABLE_HEADER_WORDS + ag.num_ranks]
    ag_gemm_intra_node_op(a, b, c, ag, order_table=table, table_header=True)
    ictx.last_round = ag.flag_round
    if env_flag("TRIDIST_VERIFY"):
        ictx.verify_hits += _verify_and_repair(a, b, c, ictx)
    return c


def i1_ag_tr(a, b, ictx):
    M = a.shape[0] * ictx.ag.num_ranks
    c = torch.empty((M, b.shape[0]), dtype=ictx.ag.output_dtype, device=a.device)
    return i1_ag_tr_op(a, b, c, ictx)


def i1_observer_read(ictx) -> List[int]:
    """Call after the round is complete on the device. Returns ``[round, order..., offsets...]``:
    the remote sources ordered by the time their shard was first seen (own rank first) and each
    source's offset in ns from the earliest stamp (-1 = not observed this round)."""
    ag = ictx.ag
    R, rank = ag.num_ranks, ag.rank
    if isinstance(ag.world, CpuWorld) or ag.arrival_ns is None:
        return [ictx.last_round] + [(rank + i) % R for i in range(R)] + [-1] * R
    stamps = ag.arrival_ns.cpu().tolist()
    seen = [(t, s) for s, t in enumerate(stamps) if s != rank and 0 < t < INT64_MAX]
    seen.sort()
    t0 = seen[0][0] if seen else 0
    order = [rank] + [s for _, s in seen] + [s for s in range(R) if s != rank and s not in [x for _, x in seen]]
    offs = [(-1 if not (s != rank and 0 < stamps[s] < INT64_MAX) else int(stamps[s] - t0)) for s in range(R)]
    return [ictx.last_round] + order + offs


def observed_straggler(ictx) -> Optional[int]:
    """The source seen last this round (input of ``StickyOrderPredictor.observe``)."""
    from ..parallel.predictor import infer_straggler
    ag = ictx.ag
    if isinstance(ag.world, CpuWorld) or ag.arrival_ns is None:
        return None
    return infer_straggler(ag.arrival_ns.cpu().tolist(), ag.rank)


def calibrate_sleep_cycles_per_us(cycles: int = 1 << 22, iters: int = 5) -> float:
    """Cycles of ``torch.cuda._sleep`` per microsecond, from event timing (median of ``iters``)."""
    torch.cuda._sleep(cycles)
    torch.cuda.synchronize()
    vals = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch.cuda._sleep(cycles)
        e1.record()
        torch.cuda.synchronize()
        vals.append(cycles / (e0.elapsed_time(e1) * 1e3))
    vals.sort()
    return vals[len(vals) // 2]
