"""GEMM+RS, windowed-pipeline entry points (reference: triton_dist/kernels/dcu/gemm_rs_v5.py:220-552).

The reference's "v5" replaces its three serial phases by a ticketed pipeline of
chunk GEMMs, per-destination pushes and slot reductions on many streams, with a
CTA budget for the reduce kernels. The base operator here is already one kernel
with per-tile tickets, owner-interleaved tile order and in-epilogue reduction, so
these entry points keep the reference's names and argument lists and run that
kernel. ``chunk_rows``, ``stage_slots``, ``comm_lanes``, ``steady_sms``, ``tail_sms``,
``tail_chunk_window`` and ``wait_mode`` are accepted and have no effect.
"""
from __future__ import annotations

import torch

from .gemm_reduce_scatter import (GemmRSContext, create_gemm_rs_intra_node_context, finalize_gemm_rs_context,
                                  gemm_rs_intra_node_op)
from ._gemm_common import gemm_nt

GemmRSv5Context = GemmRSContext


def create_gemm_rs_v5_context(max_M, N, output_dtype, rank, num_ranks, mpi=None, comm=None, chunk_rows=0,
                              stage_slots=4, comm_lanes=2, steady_sms=0, tail_sms=0, tail_chunk_window=1,
                              wait_mode=None, world=None):
    assert max_M % num_ranks == 0, "row-sharded output needs M % R == 0"
    assert N % 128 == 0 and (max_M // num_ranks) % 64 == 0
    return create_gemm_rs_intra_node_context(max_M, N, output_dtype, rank, num_ranks, mpi, comm, world=world)


def gemm_rs_v5_op(a, b, out, ctx, component="full"):
    """``out[M / R, N]`` receives this rank's rows of the reduced product.

    ``component="gemm"``: local GEMM only; the rank's own row block of its partial product is
    written to ``out`` and nothing is exchanged.
    """
    if component not in ("full", "gemm"):
        raise ValueError(f"unknown component {component!r}")
    if component == "gemm":
        m_pr = a.shape[0] // ctx.num_ranks
        if a.is_cuda:
            gemm_nt(a[ctx.rank * m_pr:(ctx.rank + 1) * m_pr], b, out=out)
        else:
            out.copy_((a[ctx.rank * m_pr:(ctx.rank + 1) * m_pr].float() @ b.float().t()).to(out.dtype))
        return out
    res = gemm_rs_intra_node_op(a, b, ctx.output_dtype, ctx.rank, ctx.num_ranks, ctx,
                                out=out if a.is_cuda else None)
    if res is not out:
        out.copy_(res)
    return out


def gemm_rs_v5(a, b, ctx):
    out = torch.empty((a.shape[0] // ctx.num_ranks, b.shape[0]), dtype=ctx.output_dtype, device=a.device)
    return gemm_rs_v5_op(a, b, out, ctx)


def finalize_gemm_rs_v5_context(ctx):
    finalize_gemm_rs_context(ctx)
