"""GEMM + reduce-scatter:  out_r = rows r of  sum_s A_s @ B_s^T   (tensor-parallel output side).

Public API follows the reference (triton_dist/kernels/dcu/gemm_reduce_scatter.py:224-300):

* ``create_gemm_rs_intra_node_context(max_M, N, output_dtype, rank, num_ranks, mpi, comm,
  fuse_scatter=True, transpose_weight=False)``
* ``gemm_rs_intra_node_op(a, b, output_dtype, rank, num_ranks, ctx)`` with ``a[M, K_loc]``,
  ``b[N, K_loc]``; returns a new ``[M / R, N]`` tensor.
* ``gemm_rs_intra_node(a, b, ctx)`` wrapper.

Two forms of the one persistent kernel, chosen per context:

switch    (on a fabric with multicast, the default there) partial tiles stay
          in the producing rank's own plane of a multicast-bound buffer; all ranks walk the
          owners' row segments in lockstep, and the communication warps of the rank that keeps a
          tile's rows read the SUM of the R partials with ``multimem.ld_reduce`` (added inside
          the NVSwitch, fp32 accumulation) and store it. No epilogue ever waits, no SM adds.
slots     tiles are visited owner by owner (rank+1 first, own rows last). The epilogue of a tile owned by another rank converts the
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
from ..utils.config import env_int, env_str
from ._gemm_common import (next_round, BM, OP_RS, SCHED_NATURAL, SCHED_SEGMENT, PlanCache, base_desc, choose_bn,
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
    mc: Optional[object] = None              # McBuffer [2][max_M, N]: this rank's partials, read through the switch
    mode: str = "auto"                       # "auto" | "slots" | "nvls"
    reduce_ctas: int = 0                     # switch form: CTAs that reduce in the steady phase (0 = all)
    reduce_tail: int = 0                     # switch form: last blocks that every CTA helps with
    round: int = 0
    plans: PlanCache = field(default_factory=PlanCache)
    order_override: Optional[list] = None

    @property
    def max_tiles(self) -> int:
        return ((self.max_M + BM - 1) // BM) * ((self.N + 127) // 128)


def create_gemm_rs_intra_node_context(max_M, N, output_dtype, rank, num_ranks, mpi=None, comm=None,
                                      fuse_scatter=True, transpose_weight=False, world=None,
                                      nvls: Optional[bool] = None):
    """Collective. ``fuse_scatter`` / ``transpose_weight`` accept only the reference's defaults.
    ``nvls`` (True / False / None = by the environment: on wherever the fabric has multicast) also allocates
    the multicast-bound partial planes of the switch-reduced form and checks them once with known
    integers."""
    if not fuse_scatter or transpose_weight:
        raise NotImplementedError("only fuse_scatter=True, transpose_weight=False are implemented")
    assert max_M % num_ranks == 0
    if world is None:
        world = default_world() or init_runtime(rank, num_ranks, comm)
    ctx = GemmRSContext(rank=rank, num_ranks=num_ranks, max_M=max_M, N=N, output_dtype=output_dtype,
                        world=world)
    if isinstance(world, CpuWorld):
        return ctx
    ctx.mode = env_str("TRIDIST_RS_MODE", "auto")
    ctx.reduce_ctas = env_int("TRIDIST_RS_REDUCE_CTAS", 0)
    ctx.reduce_tail = env_int("TRIDIST_RS_REDUCE_TAIL", 0)
    if num_ranks > 1:
        ctx.slots = world.alloc(2 * max_M * N * 2, rank)
        ctx.tile_flags = world.alloc(num_ranks * ctx.max_tiles * 4, rank)
        if nvls is None:
            nvls = ctx.mode in ("nvls", "auto")
        if nvls and (max_M // num_ranks) % BM == 0:
            ctx.mc = world.alloc_multicast(2 * max_M * N * 2)
        if ctx.mc is not None and env_int("TRIDIST_NVLS_SELFTEST", 1):
            _nvls_selftest(ctx)
        if ctx.mode == "nvls" and ctx.mc is None:
            raise RuntimeError("tridist_b200: TRIDIST_RS_MODE=nvls but no multicast buffer could be made: "
                               + str(getattr(world, "multicast_unavailable", "not a multi-process world")))
    world.host_barrier()
    return ctx


def pick_mode(ctx, M: int) -> str:
    """``local`` (one rank), ``nvls`` (partials read through the switch) or ``slots`` (peer stores)."""
    if ctx.num_ranks == 1:
        return "local"
    if ctx.mode == "slots" or ctx.mc is None or (M // ctx.num_ranks) % BM != 0:
        if ctx.mode == "nvls":
            raise RuntimeError("tridist_b200: mode 'nvls' needs a multicast buffer and rows per rank % 128 == 0")
        return "slots"
    return "nvls"


def _nvls_selftest(ctx) -> None:
    """Collective. One small reduce-scatter of known integers through the switch; if any rank sees a
    wrong value or a kernel-reported failure, all ranks drop the multicast buffer together and the
    context keeps to the peer-slot form."""
    import torch.distributed as dist
    world, R, rank = ctx.world, ctx.num_ranks, ctx.rank
    M, K = min(ctx.max_M, 128 * R), 64
    dev = torch.device("cuda", world.device)
    a = torch.full((M, K), float(rank + 1), dtype=ctx.output_dtype, device=dev)
    b = torch.ones((ctx.N, K), dtype=ctx.output_dtype, device=dev)
    expect = float(K * R * (R + 1) // 2)          # exact in fp16 and bf16 for R <= 8
    why = ""
    saved = ctx.mode
    try:
        ctx.mode = "nvls"
        for _ in range(2):                         # both parities
            out = gemm_rs_intra_node_op(a, b, ctx.output_dtype, rank, R, ctx)
            torch.cuda.synchronize()
            world.check()
            bad = int((out.float() != expect).sum().item())
            if bad:
                why = f"{bad} of {out.numel()} values differ from {expect}"
                break
    except Exception as exc:
        why = f"{type(exc).__name__}: {exc}"
        try:
            world.clear_status()
        except Exception:
            pass
    ctx.mode = saved
    ctx.plans.clear()
    verdicts = [None] * R
    dist.all_gather_object(verdicts, why, group=world.group)
    if any(verdicts):
        world.multicast_unavailable = "self-test failed: " + "; ".join(
            f"rank {r}: {v}" for r, v in enumerate(verdicts) if v)
        world.free_multicast(ctx.mc)
        ctx.mc = None


def _plan(ctx, a, b, out):
    R, rank = ctx.num_ranks, ctx.rank
    M, K = a.shape
    N = b.shape[0]
    m_pr = M // R
    bn = choose_bn(M, N, K=K)
    mode = pick_mode(ctx, M)
    # through the switch all ranks walk the same order (lockstep over the owners' segments)
    order = list(range(R)) if mode == "nvls" else (ctx.order_override or rotation_order(rank, R, 1, own_last=True))
    key = (a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
           a.dtype, bn, tuple(order), mode, ctx.reduce_ctas, ctx.reduce_tail)

    def make():
        d = base_desc(ctx.world, rank, R, a, b, out.data_ptr(), out.stride(0), M, N, K, bn, OP_RS)
        d["m_per_rank"] = m_pr
        d["sched"] = SCHED_SEGMENT if (R > 1 and m_pr % BM == 0) else SCHED_NATURAL
        d["seg_order"] = order
        if R > 1:
            half = ctx.max_M * ctx.N * 2
            d["peer_tile_flags"] = ctx.tile_flags.ptrs()
            d["ticket_stride"] = ctx.max_tiles       # one word per (source, tile) for every M
            if mode == "nvls":
                # partials stay here: every "slot" entry is this rank's own partial plane
                d["nvls"] = 1
                d["seg_interleave"] = 1
                d["peer_slots"] = [[ctx.mc.local_ptr] * R, [ctx.mc.local_ptr + half] * R]
                d["slot_stride"] = 0
                d["mc_part"] = [ctx.mc.mc_ptr, ctx.mc.mc_ptr + half]
                d["reduce_ctas"], d["reduce_tail"] = ctx.reduce_ctas, ctx.reduce_tail
            else:
                d["peer_slots"] = [ctx.slots.ptrs(0), ctx.slots.ptrs(half)]
                d["slot_stride"] = m_pr * N
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
    ctx.round = next_round(ctx.round, "reduce-scatter context")
    pid = _plan(ctx, a, b, out)
    native().gemm_plan_launch(pid, ctx.round, ctx.round & 1, 0, 0)
    return out


def gemm_rs_intra_node(a, b, ctx):
    return gemm_rs_intra_node_op(a, b, ctx.output_dtype, ctx.rank, ctx.num_ranks, ctx)


def gemm_rs_emulated(ctxs, a_list, b_list):
    outs = []
    for ctx, a, b in zip(ctxs, a_list, b_list):
        _check_args(a, b, ctx)
        ctx.round = next_round(ctx.round, "reduce-scatter context")
        outs.append(torch.empty((a.shape[0] // ctx.num_ranks, b.shape[0]), dtype=a.dtype, device=a.device))
    pids = [_plan(ctx, a, b, o) for ctx, a, b, o in zip(ctxs, a_list, b_list, outs)]
    rnd = ctxs[0].round
    native().gemm_plans_launch_emulated(pids, rnd, rnd & 1, 0)
    return outs


def finalize_gemm_rs_context(ctx) -> None:
    ctx.plans.clear()
    if ctx.mc is not None:
        ctx.world.free_multicast(ctx.mc)
        ctx.mc = None
    if ctx.slots is not None and not isinstance(ctx.world, EmulatedWorld):
        ctx.world.free(ctx.slots)
        ctx.world.free(ctx.tile_flags)
    ctx.slots = ctx.tile_flags = None
