"""Order-driven GEMM+AR carrier (reference: triton_dist/kernels/dcu/gemm_ar_pred.py:40-175).

``gemm_ar_pred_op(a, b, c, ctx, order=None, gates=())`` computes the all-reduced product
panel by panel (row panels of ``ctx.chunk_rows`` rows) in a caller-chosen order, with
optional *gates*: before a gated panel is started the stream waits until a flag word
reaches a ticket. A host thread that raises the flag after a delay turns this into the
reference's straggler-injection rig (bench/l1_pred_ar_bench.py:282-299); the predictor
experiment then measures how much earlier the non-victim panels complete when the
victim panel is ordered last. Per-panel completion events are recorded
(``task_events(ctx)``).

Tickets are keyed by execution position, not by panel id (the rule the reference
derives at gemm_ar_pred.py:107-124): every panel is one fused-kernel call and the
context's round counter advances per call, so all ranks must pass the same order.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence, Tuple

import torch

from ..parallel.runtime import CpuWorld, native
from .gemm_allreduce import gemm_ar_intra_node_op


def make_gate_flag() -> torch.Tensor:
    """A flag word in pinned host memory: kernels can poll it, a host thread can set it
    (``flag[0] = ticket``) without any CUDA call."""
    return torch.zeros(1, dtype=torch.int32).pin_memory()


def chunk_rows_of(ctx) -> int:
    return int(getattr(ctx, "chunk_rows", 0) or ctx.M_PER_CHUNK)


def task_events(ctx) -> List[Tuple[torch.cuda.Event, torch.cuda.Event]]:
    """(start, end) events of the panels of the last ``gemm_ar_pred_op`` call, by panel id."""
    return getattr(ctx, "_task_events", [])


def gemm_ar_pred_op(a, b, c, ctx, order: Optional[Sequence[int]] = None,
                    gates: Iterable[Tuple[int, int, int]] = ()):
    """``c = sum_r a_r @ b_r.T`` with a chosen panel order.

    order  permutation of ``range(n_tasks)`` (natural order if None); identical on all ranks
    gates  iterable of ``(task_id, flag_address, expected_ticket)``; the wait is bounded by
           the world's wait limit and reports through the status plane when it runs out
    """
    M, K = a.shape
    rows_per = chunk_rows_of(ctx)
    n_tasks = (M + rows_per - 1) // rows_per
    if order is None:
        order = list(range(n_tasks))
    assert sorted(order) == list(range(n_tasks)), "order must permute tasks"
    gate_map = {int(t): (int(va), int(exp)) for t, va, exp in gates}
    cpu = isinstance(ctx.world, CpuWorld)
    events: List = [None] * n_tasks
    for task in order:
        r0 = task * rows_per
        rows = min(rows_per, M - r0)
        if task in gate_map and not cpu:
            va, exp = gate_map[task]
            w = ctx.world
            native().wait_flag_test(va, exp, w.status_dev, w.abort_word, w.timeout_ns)
        if not cpu:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        gemm_ar_intra_node_op(a[r0:r0 + rows], b, c[r0:r0 + rows], ctx)
        if not cpu:
            e1.record()
            events[task] = (e0, e1)
    ctx._task_events = events
    return c
