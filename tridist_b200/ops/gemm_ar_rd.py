"""GEMM+AR, "recursive doubling" entry points (reference: triton_dist/kernels/dcu/gemm_ar_rd.py:268-522).

The reference exchanges row panels with XOR partners in log2(R) rounds because its
fabric cannot sustain a full-mesh fan-out. NVSwitch gives every pair of GPUs full
bandwidth, so the fused one-shot / two-shot kernel of ``gemm_allreduce`` is used
instead; the names, argument lists, the power-of-two rank check and the
decomposition modes of the reference are kept. ``chunk_rows`` (or ``target_chunks`` /
``min_chunk_rows``, from which the reference derives it) sets the row-panel size of the
order-driven carrier ``gemm_ar_pred_op``; inside one fused call there are no panels, no
partner rounds and no staging slots, so ``stage_slots`` and ``wait_mode`` have no effect
(a warning says so once when a non-default value is passed).
"""
from __future__ import annotations

from ._gemm_common import warn_ignored
from .gemm_allreduce import (GemmARContext, create_gemm_ar_intra_node_context, finalize_gemm_ar_context,
                             gemm_ar_intra_node, gemm_ar_intra_node_op)

GemmARRDContext = GemmARContext
MAX_TICKETS = 1 << 20


def create_gemm_ar_rd_context(max_M, N, input_dtype, output_dtype, rank, num_ranks, mpi=None, comm=None,
                              chunk_rows=0, target_chunks=4, min_chunk_rows=512, stage_slots=4,
                              wait_mode=None, world=None):
    assert num_ranks & (num_ranks - 1) == 0, "recursive doubling needs 2^k ranks"
    assert input_dtype == output_dtype, "panels are exchanged in output dtype"
    assert N % 128 == 0 and max_M % 64 == 0
    ctx = create_gemm_ar_intra_node_context(max_M, N, input_dtype, output_dtype, rank, num_ranks, mpi, comm,
                                            M_PER_CHUNK=64, world=world)
    # panel rows of the order-driven carrier (reference rule: about target_chunks panels, not
    # below min_chunk_rows, 64-row aligned: gemm_ar_rd.py:317-323 there)
    rows = int(chunk_rows) if chunk_rows else max(min_chunk_rows, max_M // max(1, target_chunks))
    rows = max(64, min(rows, max_M) // 64 * 64)
    ctx.chunk_rows = rows
    warn_ignored("create_gemm_ar_rd_context", stage_slots=(stage_slots, 4), wait_mode=(wait_mode, None))
    return ctx


def gemm_ar_rd_op(a, b, c, ctx, component="full"):
    return gemm_ar_intra_node_op(a, b, c, ctx, component=component)


def gemm_ar_rd(a, b, ctx):
    return gemm_ar_intra_node(a, b, ctx)


def finalize_gemm_ar_rd_context(ctx):
    finalize_gemm_ar_context(ctx)
