"""GEMM+RS, windowed-pipeline entry points (reference: triton_dist/kernels/dcu/gemm_rs_v5.py:220-552).

The reference's "v5" replaces its three serial phases by a ticketed pipeline of
chunk GEMMs, per-destination pushes and slot reductions on many streams, with a
CTA budget for the reduce kernels. The base operator here is already one kernel
with per-tile tickets, lockstep owner order and owner-side reduction, so these entry
points keep the reference's names and argument lists and run that kernel, with the
reference's reduce budget mapped onto it: ``steady_sms`` CTAs reduce the owner's blocks
while tiles are still being computed, and for the last ``tail_chunk_window`` chunks
(``chunk_rows`` rows each) every CTA helps (``tail_sms`` = 0 or the whole grid; other
values are rounded to the whole grid). The budget applies to the switch-reduced form
(the default wherever the fabric has multicast). ``stage_slots``, ``comm_lanes`` and
``wait_mode`` have no counterpart (no slot window, no copy lanes, in-kernel bounded waits);
a warning says so once when a non-default value is passed.
"""
from __future__ import annotations

import torch

from .gemm_reduce_scatter import (GemmRSContext, create_gemm_rs_intra_node_context, finalize_gemm_rs_context,
                                  gemm_rs_intra_node_op)
from ._gemm_common import gemm_nt, warn_ignored

GemmRSv5Context = GemmRSContext


def create_gemm_rs_v5_context(max_M, N, output_dtype, rank, num_ranks, mpi=None, comm=None, chunk_rows=0,
                              stage_slots=4, comm_lanes=2, steady_sms=0, tail_sms=0, tail_chunk_window=1,
                              wait_mode=None, world=None):
    assert max_M % num_ranks == 0, "row-sharded output needs M % R == 0"
    assert N % 128 == 0 and (max_M // num_ranks) % 64 == 0
    ctx = create_gemm_rs_intra_node_context(max_M, N, output_dtype, rank, num_ranks, mpi, comm, world=world)
    ctx.reduce_ctas = int(steady_sms)
    rows = int(chunk_rows) if chunk_rows else 0
    # blocks of 128 rows x 256 columns in the last `tail_chunk_window` chunks of the owner's rows
    ctx.reduce_tail = ((max(rows, 128) // 128) * ((N + 255) // 256) * int(tail_chunk_window)) if steady_sms else 0
    warn_ignored("create_gemm_rs_v5_context", stage_slots=(stage_slots, 4), comm_lanes=(comm_lanes, 2),
                 wait_mode=(wait_mode, None))
    return ctx


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
