"""AG+GEMM, "tile-ready" entry points (reference: triton_dist/kernels/dcu/gemm_ag_tr.py:234-529).

The reference re-designs its all-gather as a barrier-free, ticketed, chunk-major
*pull* pipeline on several streams: every rank stages its shard, tells the peers chunk
by chunk that it is there ("arrive"), the peers copy it out and raise their own "ready"
tickets for the consumer. The same transport runs here inside the one fused kernel
(``transport="pull"``, the default of these entry points): the transfer CTAs stage,
signal, pull through their copy engines and raise the ready tickets the producer warp
waits on; ``transport="push"`` selects the base operator's push instead (one hop less).

``chunk_rows`` sets the ticket granularity, ``comm_lanes`` the number of transfer CTAs
(8 per lane; 2 lanes = the default of 16). ``wait_mode`` has no counterpart: every wait is
an in-kernel bounded spin.
"""
from __future__ import annotations

import torch

from ._gemm_common import warn_ignored
from .all_gather_gemm import (ag_gemm_intra_node_op, create_ag_gemm_intra_node_context,
                              finalize_ag_gemm_context)

GemmAGTRContext = None  # set below (alias of the base context class)


def _auto_chunk_rows(m_per_rank: int, target_chunks_per_rank: int = 2, min_chunk_rows: int = 1024) -> int:
    """Largest 128-aligned divisor of the shard giving about ``target`` chunks per rank."""
    want = max(min_chunk_rows, m_per_rank // max(1, target_chunks_per_rank))
    rows = (min(want, m_per_rank) // 128) * 128
    while rows >= 128 and m_per_rank % rows != 0:
        rows -= 128
    return rows if rows >= 128 else m_per_rank


def create_gemm_ag_tr_context(max_M, K, input_dtype, output_dtype, rank, num_ranks, mpi=None, comm=None,
                              chunk_rows=0, comm_lanes=2, wait_mode=None, world=None, transport="pull"):
    assert max_M % num_ranks == 0, "gather needs M % R == 0"
    m_pr = max_M // num_ranks
    assert K % 16 == 0 and input_dtype == output_dtype
    rows = chunk_rows or _auto_chunk_rows(m_pr)
    if m_pr % 128 != 0:
        rows = m_pr
    ctx = create_ag_gemm_intra_node_context(max_M, K, input_dtype, output_dtype, rank, num_ranks, mpi, comm,
                                            M_PER_CHUNK=rows, world=world, transport=transport)
    ctx.chunk_rows = rows
    assert transport in ("pull", "push", "mc", "auto")
    if transport in ("pull", "push"):
        ctx.transport = transport
    if comm_lanes != 2:
        ctx.push_ctas = max(2, 8 * int(comm_lanes))
    warn_ignored("create_gemm_ag_tr_context", wait_mode=(wait_mode, None))
    return ctx


def gemm_ag_tr_op(a, b, c, ctx, component="full"):
    """``component="gemm"`` multiplies the workspace of the last full call (no communication)."""
    if component not in ("full", "gemm"):
        raise ValueError(f"unknown component {component!r}")
    return ag_gemm_intra_node_op(a, b, c, ctx, skip_comm=(component == "gemm"))


def gemm_ag_tr(a, b, ctx):
    M = a.shape[0] * ctx.num_ranks
    c = torch.empty((M, b.shape[0]), dtype=ctx.output_dtype, device=a.device)
    return gemm_ag_tr_op(a, b, c, ctx)


def finalize_gemm_ag_tr_context(ctx):
    finalize_ag_gemm_context(ctx)


from .all_gather_gemm import AllGatherGEMMTensorParallelContext as GemmAGTRContext  # noqa: E402,F811
