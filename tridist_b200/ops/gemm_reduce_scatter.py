"""GEMM + reduce-scatter:  out_r = rows r of  sum_s A_s @ B_s^T   (tensor-parallel output side).

Public API follows the reference (triton_dist/kernels/dcu/gemm_reduce_scatter.py:224-300):

* ``create_gemm_rs_intra_node_context(max_M, N, output_dtype, rank, num_ranks, mpi, comm,
  fuse_scatter=True, transpose_weight=False)``
* ``gemm_rs_intra_node_op(a, b, output_dtype, rank, num_ranks, ctx)`` with ``a[M, K_loc]``,
  ``b[N, K_loc]``; returns a new ``[M / R, N]`` tensor.
* ``gemm_rs_intra_node(a, b, ctx)`` wrapper.

Mechanism: one persistent kernel. Tiles are visited owner by owner (rank+1
first, own rows last). The epilogue of a tile owned by another rank converts the
fp32 accumulator and stores it directly into that rank's slot ``[source, row, col]``
over NVLink, then raises the tile's ticket there; the epilogue of an own tile
waits for the R-1 tickets, adds the peers' partials from its local slots to the
fp32 accumulator in a fixed source order and writes the final rows. The
reference runs three serial phases with two global barriers and reduces in the
output dtype (gemm_reduce_scatter.py:113-135, 224-243); here there is no
barrier, no scatter pass, no separate reduce pass, and the sum is fp32.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..parallel import cpu_backend
from ..parallel.runtime import (CpuWorld, EmulatedWorld, SymmBuffer, default_world, init_runtime,
                                native)
from ._gemm_common import (BM, OP_RS, SCHED_NATURAL, SCHED_SEGMENT, PlanCache, base_desc, choose_bn,
                           debug_check, rotation_order, tensor_extent_bytes)


@dataclass
class GemmRSContext:
    rank: int
    num_ranks: int
    max_M: int
    N: int
    output_dtype: torch.dtype
    world: object
    slots: Optional[SymmBuffer] = None       # [2][R, max_M / R, N] partial tiles, by source
    tile_flags: Optional[SymmBuffer] = None  # u32 [R, max_tiles] tickets, by source
    round: int = 0
    plans: PlanCache = field(default_factory=PlanCache)
    order_override: Optional[list] = None

    @property
    def max_tiles(self) -> int:
        return ((self.max_M + BM - 1) // BM) * ((self.N + 127) // 128)


def create_gemm_rs_intra_node_context(max_M, N, output_dtype, rank, num_ranks, mpi=None, comm=None,
                                      fuse_scatter=True, transpose_weight=False, world=None):
    """Collective. ``fuse_scatter`` / ``transpose_weight`` accept only the reference's defaults."""
    if not fuse_scatter or transpose_weight:
        raise NotImplementedError("only fuse_scatter=True, transpose_weight=False are implemented")
    assert max_M % num_ranks == 0
    if world is None:
        world = default_world() or init_runtime(rank, num_ranks, comm)
    ctx = GemmRSContext(rank=rank, num_ranks=num_ranks, max_M=max_M, N=N, output_dtype=output_dtype,
                        world=world)
    if isinstance(world, CpuWorld):
        return ctx
    if num_ranks > 1:
        ctx.slots = world.alloc(2 * max_M * N * 2, rank)
        ctx.tile_flags = world.alloc(num_ranks * ctx.max_tiles * 4, rank)
    world.host_barrier()
    return ctx


def _plan(ctx, a, b, out):
    R, rank = ctx.num_ranks, ctx.rank
    M, K = a.shape
    N = b.shape[0]
    m_pr = M // R
    bn = choose_bn(M, N)
    order = ctx.order_override or rotation_order(rank, R, 1, own_last=True)
    key = (a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
           a.dtype, bn, tuple(order))

    def make():
        d = base_desc(ctx.world, rank, R, a, b, out.data_ptr(), out.stride(0), M, N, K, bn, OP_RS)
        d["m_per_rank"] = m_pr
        d["sched"] = SCHED_SEGMENT if (R > 1 and m_pr % BM == 0) else SCHED_NATURAL
        d["seg_order"] = order
        if R > 1:
            half = ctx.max_M * ctx.N * 2
            d["peer_slots"] = [ctx.slots.ptrs(0), ctx.slots.ptrs(half)]
            d["slot_stride"] = m_pr * N
            d["peer_tile_flags"] = ctx.tile_flags.ptrs()
            d["ticket_stride"] = ctx.max_tiles       # one word per (source, tile) for every M
            debug_check(d, c_bytes=tensor_extent_bytes(out), slot_bytes=half,
                        tile_flag_words=ctx.tile_flags.nbytes // 4)
        else:
            debug_check(d, c_bytes=tensor_extent_bytes(out))
        return native().gemm_plan_create(d)

    return ctx.plans.get(key, make)


def _check_args(a, b, ctx):
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K and a.dtype == b.dtype
    assert M <= ctx.max_M and N == ctx.N, "shape exceeds the context"
    assert M % ctx.num_ranks == 0 and M % 128 == 0 and N % 128 == 0 and K % 16 == 0
    assert a.stride(1) == 1 and b.stride(1) == 1


def gemm_rs_intra_node_op(a, b, output_dtype, rank, num_ranks, ctx, out: Optional[torch.Tensor] = None):
    """Returns ``[M / R, N]``: this rank's rows of the sum over ranks of ``a @ b.T``."""
    if isinstance(ctx.world, CpuWorld):
        return cpu_backend.gemm_rs(a, b, output_dtype, ctx)
    _check_args(a, b, ctx)
    assert output_dtype == a.dtype, "the fused kernel emits the input dtype"
    M = a.shape[0]
    if out is None:
        out = torch.empty((M // num_ranks, b.shape[0]), dtype=output_dtype, device=a.device)
    ctx.round += 1
    pid = _plan(ctx, a, b, out)
    native().gemm_plan_launch(pid, ctx.round, ctx.round & 1, 0, 0)
    return out


def gemm_rs_intra_node(a, b, ctx):
    return gemm_rs_intra_node_op(a, b, ctx.output_dtype, ctx.rank, ctx.num_ranks, ctx)


def gemm_rs_emulated(ctxs, a_list, b_list):
    outs = []
    for ctx, a, b in zip(ctxs, a_list, b_list):
        _check_args(a, b, ctx)
        ctx.round += 1
        outs.append(torch.empty((a.shape[0] // ctx.num_ranks, b.shape[0]), dtype=a.dtype, device=a.device))
    pids = [_plan(ctx, a, b, o) for ctx, a, b, o in zip(ctxs, a_list, b_list, outs)]
    rnd = ctxs[0].round
    native().gemm_plans_launch_emulated(pids, rnd, rnd & 1, 0)
    return outs


def finalize_gemm_rs_context(ctx) -> None:
    ctx.plans.clear()
    if ctx.slots is not None and not isinstance(ctx.world, EmulatedWorld):
        ctx.world.free(ctx.slots)
        ctx.world.free(ctx.tile_flags)
    ctx.slots = ctx.tile_flags = None
