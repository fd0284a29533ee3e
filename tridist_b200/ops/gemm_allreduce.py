"""GEMM + all-reduce:  C = sum_r A_r @ B_r^T, full C on every rank (K sharded).

Public API follows the reference (triton_dist/kernels/dcu/gemm_allreduce.py:250-449):

* ``create_gemm_ar_intra_node_context(max_M, N, input_dtype, output_dtype, rank, num_ranks,
  mpi, comm, M_PER_CHUNK=512, gemm_stream=None, ar_stream=None)``
* ``gemm_ar_intra_node_op(a, b, c, ctx, component="full")`` with ``a[M, K_loc]``, ``b[N, K_loc]``,
  ``c[M, N]``; ``component`` in {"full", "gemm", "push"} for the decomposition
* ``gemm_ar_intra_node(a, b, ctx)`` allocates c.

Two fused algorithms live in the one persistent kernel and are chosen by size:

one-shot  every epilogue stores its 16-bit partial tile into all ranks' slots and
          raises the tile ticket; every rank then sums the R partials of the tile
          in a fixed order (bit-identical result everywhere). One NVLink hop;
          best for small M (latency-bound decode shapes).
two-shot  tile t is owned by rank t % R. Every rank stores its partial into the
          owner's slot; the owner's communication warps add the R partials in fp32 and
          broadcast the reduced tile into every rank's result buffer. 2(R-1)/R of
          the one-shot traffic; best for large M.
nvls      two-shot with the NVSwitch doing the arithmetic: partial tiles stay in the
          producing rank's own memory, the owner reads the SUM of the R copies with
          ``multimem.ld_reduce`` (added inside the switch, fp32 accumulation) and writes the
          result to all ranks with one ``multimem.st``. Per rank (R-1)/R + 1/R of the
          data leaves the GPU instead of 2(R-1)/R, and no SM adds anything. Needs a
          multicast-capable buffer (``ProcessWorld.alloc_multicast``), which the context
          allocates by default at three or more ranks (``nvls=False``, ``TRIDIST_NVLS=0``
          or a fabric without multicast support leave it out) and checks once with known
          integers before use. With it, ``auto`` takes this path for every size
          (``TRIDIST_AR_NVLS_MIN_BYTES`` raises the threshold): at 4 GPUs it is ahead of
          both peer-store algorithms from M = 128 to M = 4096 (K 28672, N 8192). At two
          ranks one-shot moves the same bytes with one hop less and stays the choice.
          The summation order inside the switch is not specified, but each tile is
          reduced once, by its owner, so all ranks still hold bit-identical results.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..parallel import cpu_backend
from ..parallel.runtime import (CpuWorld, EmulatedWorld, SymmBuffer, default_world, init_runtime,
                                native)
from ..utils.config import env_int, env_str
from ._gemm_common import (next_round, BM, OP_AR1, OP_AR2, OP_PLAIN, SCHED_STRIDED, PlanCache,
                           base_desc, choose_bn, debug_check, rotation_order, tensor_extent_bytes)


@dataclass
class GemmARContext:
    rank: int
    num_ranks: int
    max_M: int
    N: int
    input_dtype: torch.dtype
    output_dtype: torch.dtype
    M_PER_CHUNK: int
    world: object
    slots: Optional[SymmBuffer] = None       # [2][R, max_M, N] partials by source
    res: Optional[SymmBuffer] = None         # [2][max_M, N] reduced result (two-shot)
    tile_flags: Optional[SymmBuffer] = None  # u32 [R, max_tiles]
    res_flags: Optional[SymmBuffer] = None   # u32 [R, max_tiles], by owner
    mc: Optional[object] = None              # McBuffer [part 0 | part 1 | res 0 | res 1], each max_M * N
    flag_round: int = 0
    plans: PlanCache = field(default_factory=PlanCache)
    mode: str = "auto"

    @property
    def max_tiles(self) -> int:
        return ((self.max_M + BM - 1) // BM) * ((self.N + 127) // 128)

    def symm_output(self, M: int, parity: Optional[int] = None) -> torch.Tensor:
        """The [M, N] view of the NEXT call's result buffer. Passing it as ``c`` lets the
        two-shot kernel deliver peers' reduced tiles straight into ``c`` (no copy)."""
        if parity is None:
            parity = (self.flag_round + 1) & 1
        plane = self.max_M * self.N * 2
        if pick_mode(self, M) == "nvls":
            return self.mc.tensor(self.output_dtype, (M, self.N), (2 + parity) * plane, rank=self.rank)
        return self.res.tensor(self.output_dtype, (M, self.N), parity * plane, rank=self.rank)


def create_gemm_ar_intra_node_context(max_M, N, input_dtype, output_dtype, rank, num_ranks, mpi=None,
                                      comm=None, M_PER_CHUNK=512, gemm_stream=None, ar_stream=None,
                                      world=None, nvls: Optional[bool] = None):
    """Collective. Allocates partial-slot, result and ticket planes on the symmetric heap, and
    (``nvls``: True / False / None = as the environment says) the multicast-bound planes of the
    switch-reduced algorithm."""
    assert input_dtype == output_dtype, "input and output dtype must match"
    M_PER_CHUNK = min(M_PER_CHUNK, max_M)
    assert max_M % M_PER_CHUNK == 0 and M_PER_CHUNK % 64 == 0 and N % 128 == 0
    assert num_ranks * max_M * N < 2 ** 31
    if world is None:
        world = default_world() or init_runtime(rank, num_ranks, comm)
    ctx = GemmARContext(rank=rank, num_ranks=num_ranks, max_M=max_M, N=N, input_dtype=input_dtype,
                        output_dtype=output_dtype, M_PER_CHUNK=M_PER_CHUNK, world=world,
                        mode=env_str("TRIDIST_AR_MODE", "auto"))
    if isinstance(world, CpuWorld):
        return ctx
    if num_ranks > 1:
        ctx.slots = world.alloc(2 * num_ranks * max_M * N * 2, rank)
        ctx.res = world.alloc(2 * max_M * N * 2, rank)
        ctx.tile_flags = world.alloc(num_ranks * ctx.max_tiles * 4, rank)
        ctx.res_flags = world.alloc(num_ranks * ctx.max_tiles * 4, rank)
        if nvls is None:
            nvls = ctx.mode == "nvls" or (ctx.mode == "auto" and num_ranks >= 3)
        if nvls:
            ctx.mc = world.alloc_multicast(4 * max_M * N * 2)
        if ctx.mc is not None and env_int("TRIDIST_NVLS_SELFTEST", 1):
            _nvls_selftest(ctx)
        if ctx.mode == "nvls" and ctx.mc is None:
            raise RuntimeError("tridist_b200: TRIDIST_AR_MODE=nvls but no multicast buffer could be made: "
                               + str(getattr(world, "multicast_unavailable", "not a multi-process world")))
    world.host_barrier()
    return ctx


def _nvls_selftest(ctx) -> None:
    """Collective. One small all-reduce of known integers through the switch path; if any rank
    sees a wrong value or a kernel-reported failure, all ranks drop the multicast buffer together
    and the context keeps to the peer-store algorithms."""
    import torch.distributed as dist
    world, R, rank = ctx.world, ctx.num_ranks, ctx.rank
    M, K = min(ctx.max_M, 128), 64
    dev = torch.device("cuda", world.device)
    a = torch.full((M, K), float(rank + 1), dtype=ctx.input_dtype, device=dev)
    b = torch.ones((ctx.N, K), dtype=ctx.input_dtype, device=dev)
    expect = float(K * R * (R + 1) // 2)          # exact in fp16 and bf16 for R <= 8
    why = ""
    saved_mode = ctx.mode
    try:
        ctx.mode = "nvls"
        for _ in range(2):                         # both parities
            c = torch.empty((M, ctx.N), dtype=ctx.output_dtype, device=dev)
            gemm_ar_intra_node_op(a, b, c, ctx)
            torch.cuda.synchronize()
            world.check()
            bad = int((c.float() != expect).sum().item())
            if bad:
                why = f"{bad} of {c.numel()} values differ from {expect}"
                break
    except Exception as exc:
        why = f"{type(exc).__name__}: {exc}"
        try:
            world.clear_status()
        except Exception:
            pass
    ctx.mode = saved_mode
    ctx.plans.clear()
    verdicts = [None] * R
    dist.all_gather_object(verdicts, why, group=world.group)
    if any(verdicts):
        world.multicast_unavailable = "self-test failed: " + "; ".join(
            f"rank {r}: {v}" for r, v in enumerate(verdicts) if v)
        world.free_multicast(ctx.mc)
        ctx.mc = None


def pick_mode(ctx, M: int) -> str:
    if ctx.num_ranks == 1:
        return "local"
    if ctx.mode == "nvls" and ctx.mc is None:
        raise RuntimeError("tridist_b200: mode 'nvls' needs a context created with a multicast buffer "
                           "(nvls=True on a fabric with multicast support)")
    if ctx.mode in ("one_shot", "two_shot", "nvls"):
        return ctx.mode
    if ctx.mc is not None and ctx.num_ranks >= 3 and \
            M * ctx.N * 2 >= env_int("TRIDIST_AR_NVLS_MIN_BYTES", 0):
        return "nvls"
    if ctx.num_ranks == 2:
        return "one_shot"        # same traffic as two-shot at two ranks, one hop less
    limit = env_int("TRIDIST_AR_ONE_SHOT_BYTES", 4 << 20)
    return "one_shot" if M * ctx.N * 2 <= limit else "two_shot"


def _plan(ctx, a, b, c, mode, parity):
    R, rank = ctx.num_ranks, ctx.rank
    M, K = a.shape
    N = b.shape[0]
    bn = choose_bn(M, N, K=K if ctx.num_ranks == 1 else 0)   # (wide tiles halve the CTAs that publish and reduce)
    res_is_c = 0
    plane = ctx.max_M * ctx.N * 2
    if mode in ("two_shot", "nvls"):
        res_ptr = (ctx.res.local_ptr + parity * plane) if mode == "two_shot" else \
            (ctx.mc.local_ptr + (2 + parity) * plane)
        res_is_c = 1 if (c.data_ptr() == res_ptr and c.stride(0) == N) else 0
    key = (a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, a.stride(0), b.stride(0), c.stride(0),
           a.dtype, bn, mode, res_is_c, parity if res_is_c else -1)

    def make():
        op = {"local": OP_PLAIN, "gemm": OP_PLAIN, "one_shot": OP_AR1, "two_shot": OP_AR2,
              "nvls": OP_AR2}[mode]
        d = base_desc(ctx.world, rank, R, a, b, c.data_ptr(), c.stride(0), M, N, K, bn, op)
        if mode == "nvls":
            # partials stay here: every "slot" entry is this rank's own partial plane
            d["nvls"] = 1
            d["peer_slots"] = [[ctx.mc.local_ptr] * R, [ctx.mc.local_ptr + plane] * R]
            d["slot_stride"] = 0
            d["ticket_stride"] = ctx.max_tiles
            d["mc_part"] = [ctx.mc.mc_ptr, ctx.mc.mc_ptr + plane]
            d["mc_res"] = [ctx.mc.mc_ptr + 2 * plane, ctx.mc.mc_ptr + 3 * plane]
            d["peer_tile_flags"] = ctx.tile_flags.ptrs()
        elif op in (OP_AR1, OP_AR2):
            half = R * ctx.max_M * ctx.N * 2
            d["peer_slots"] = [ctx.slots.ptrs(0), ctx.slots.ptrs(half)]
            d["slot_stride"] = M * N
            d["peer_tile_flags"] = ctx.tile_flags.ptrs()
            d["ticket_stride"] = ctx.max_tiles       # one word per (source, tile) for every M
        if op in (OP_AR1, OP_AR2) and ((M + 255) // 256) * ((N + 255) // 256) <= 16 * 74:
            # Few rounds of tiles: 256 x 256 pair tiles instead of 512 x 256. The reduce of a tile
            # starts when the tile is done, so twice as many, half as long rounds hide more of the
            # all-reduce behind the mainloop than the wide tile saves in operand traffic
            # (4 GPUs, K 28672, N 8192: M = 1024 0.151 ms against 0.169, M = 4096 0.428 against 0.445).
            d["allow_wide"] = 0
        if op == OP_AR2:
            d["sched"] = SCHED_STRIDED
            d["seg_order"] = rotation_order(rank, R, 1, own_last=True)
            d["strided_interleave"] = 0 if env_str("TRIDIST_AR2_ORDER", "interleave") == "own_last" else 1
            if mode == "nvls":
                d["peer_res"] = [ctx.mc.ptrs(2 * plane), ctx.mc.ptrs(3 * plane)]
            else:
                d["peer_res"] = [ctx.res.ptrs(0), ctx.res.ptrs(plane)]
            d["peer_res_flags"] = ctx.res_flags.ptrs()
            d["res_is_c"] = res_is_c
        ext = dict(c_bytes=tensor_extent_bytes(c))
        if op in (OP_AR1, OP_AR2):
            ext.update(slot_bytes=plane if mode == "nvls" else R * plane, tile_flag_words=ctx.tile_flags.nbytes // 4)
        if op == OP_AR2:
            ext.update(res_bytes=plane, res_flag_words=ctx.res_flags.nbytes // 4)
        debug_check(d, **ext)
        return native().gemm_plan_create(d)

    return ctx.plans.get(key, make)


def _check_args(a, b, c, ctx):
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K and a.dtype == ctx.input_dtype and b.dtype == ctx.input_dtype
    assert M <= ctx.max_M and N == ctx.N, "shape exceeds the context"
    assert M % 64 == 0 and K % 16 == 0
    assert c.shape[0] == M and c.shape[1] == N and c.stride(1) == 1
    assert a.stride(1) == 1 and b.stride(1) == 1


def gemm_ar_intra_node_op(a, b, c, ctx, component="full"):
    """``c[M, N] = sum over ranks of a @ b.T`` (replicated).

    ``component="gemm"`` runs the local GEMM only (partial result in c, no
    communication); ``component="push"`` runs the GEMM and publishes the partial
    tiles with their tickets but reduces nothing (c is left untouched) -- the
    "GEMM + push" term of the reference's residue decomposition
    (gemm_allreduce.py:330-338 there). With one rank both are the local GEMM.
    """
    if component not in ("full", "gemm", "push"):
        raise ValueError(f"unknown component {component!r}")
    if isinstance(ctx.world, CpuWorld):
        if component == "gemm":
            c.copy_((a.float() @ b.float().t()).to(c.dtype))
            return c
        return cpu_backend.gemm_ar(a, b, c, ctx)
    _check_args(a, b, c, ctx)
    mode = "gemm" if component == "gemm" else pick_mode(ctx, a.shape[0])
    if mode not in ("gemm", "local"):
        ctx.flag_round = next_round(ctx.flag_round, "all-reduce context")
    rnd = max(ctx.flag_round, 1)
    pid = _plan(ctx, a, b, c, mode, rnd & 1)
    publish_only = component == "push" and mode not in ("gemm", "local")
    native().gemm_plan_launch(pid, rnd, rnd & 1, 0, 4 if publish_only else 0)
    return c


def gemm_ar_intra_node(a, b, ctx):
    """Allocating wrapper. With the two-shot algorithm the returned tensor is a view of the
    context's symmetric result buffer (valid until the second next call on this context)."""
    M = a.shape[0]
    if (not isinstance(ctx.world, CpuWorld)) and pick_mode(ctx, M) in ("two_shot", "nvls"):
        c = ctx.symm_output(M)
    else:
        c = torch.empty((M, b.shape[0]), dtype=ctx.output_dtype, device=a.device)
    return gemm_ar_intra_node_op(a, b, c, ctx)


def gemm_ar_emulated(ctxs, a_list, b_list, c_list, mode="one_shot"):
    for ctx, a, b, c in zip(ctxs, a_list, b_list, c_list):
        _check_args(a, b, c, ctx)
        ctx.flag_round = next_round(ctx.flag_round, "all-reduce context")
    rnd = ctxs[0].flag_round
    pids = [_plan(ctx, a, b, c, mode, rnd & 1) for ctx, a, b, c in zip(ctxs, a_list, b_list, c_list)]
    native().gemm_plans_launch_emulated(pids, rnd, rnd & 1, 0)
    return c_list


def finalize_gemm_ar_context(ctx) -> None:
    ctx.plans.clear()
    if ctx.mc is not None:
        ctx.world.free_multicast(ctx.mc)
        ctx.mc = None
    if ctx.slots is not None and not isinstance(ctx.world, EmulatedWorld):
        for buf in (ctx.slots, ctx.res, ctx.tile_flags, ctx.res_flags):
            ctx.world.free(buf)
    ctx.slots = ctx.res = ctx.tile_flags = ctx.res_flags = None
