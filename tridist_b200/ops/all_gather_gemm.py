"""All-gather + GEMM:  C = allgather_M(A) @ B^T   (tensor/sequence parallel input side).

Public API and semantics follow the reference
(triton_dist/kernels/dcu/all_gather_gemm.py:317-497):

* ``create_ag_gemm_intra_node_context(max_M, K, input_dtype, output_dtype, rank,
  num_ranks, mpi, comm, M_PER_CHUNK=1024, ag_stream=None, gemm_stream=None)``
* ``ag_gemm_intra_node_op(a, b, c, ctx, skip_comm=False)`` with ``a[M_pr, K]`` this
  rank's shard, ``b[N_pr, K]`` this rank's weight, ``c[M, N_pr]`` caller-allocated;
  row block s of C comes from rank s's shard.
* ``ag_gemm_intra_node(a, b, transe_b, ctx)`` allocates C.

What differs is the mechanism: one persistent sm_100a kernel per call. Its
communication warps move the local shard into every peer's workspace and raise a
per-(source, row block) ticket; its TMA warp waits for the ticket of a remote row block,
then loads it from the local workspace; tcgen05 tiles run own rows first, then sources in
arrival order. There is no host-side synchronisation and no global barrier: the workspace
is double-buffered by call parity.

Transports (``transport=`` / ``TRIDIST_AG_TRANSPORT``; ``auto`` = ``push``):

  mc    the workspace is bound to an NVSwitch multicast object and the shard leaves as
        ``multimem.st``: one store reaches every rank, so a rank sends its shard once instead of
        once per peer; the communication warps of a few CTAs do it (about 105 GB/s per GPU), and
        those CTAs join the GEMM when their part is out
  push  bulk copies (16 KB pieces through a shared-memory ring) into each peer's workspace by a
        few CTAs that join the GEMM late
  pull  every rank stages its shard in its own workspace, the consumers copy it out of the peers'
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..parallel import cpu_backend
from ..parallel.runtime import (CpuWorld, EmulatedWorld, SymmBuffer, default_world, init_runtime,
                                native)
from ..utils.config import env_int, env_str
from ._gemm_common import (next_round, BM, EPI_SWIGLU, OP_AG, SCHED_NATURAL, SCHED_SEGMENT, PlanCache,
                           base_desc, choose_bn, debug_check, rotation_order, tensor_extent_bytes)

_CONSUMER_BLOCK_M = 128
_CONSUMER_BLOCK_N = 128


@dataclass
class AllGatherGEMMTensorParallelContext:
    rank: int
    num_ranks: int
    max_M: int
    K: int
    input_dtype: torch.dtype
    output_dtype: torch.dtype
    M_PER_CHUNK: int
    world: object
    ws: Optional[SymmBuffer] = None          # [2][max_M, K] gathered A, double-buffered
    flags: Optional[SymmBuffer] = None       # u32 [R, max_chunks] tickets, indexed by source
    arrive: Optional[SymmBuffer] = None      # u32 [R, max_chunks] "source staged its chunk" (pull transport)
    transport: str = "push"                  # "mc" | "push" | "pull"
    mc: Optional[object] = None              # McBuffer behind ws when the workspace is multicast-bound
    push_ctas: int = 0                       # CTAs that carry the transfer (0 = chosen from the shape)
    counters: Optional[torch.Tensor] = None  # local part counters of the transfer
    arrival_ns: Optional[torch.Tensor] = None  # int64 [R] first-seen arrival stamps (observer)
    flag_round: int = 0
    ag_stream: Optional[torch.cuda.Stream] = None
    gemm_stream: Optional[torch.cuda.Stream] = None
    plans: PlanCache = field(default_factory=PlanCache)
    observe: bool = False
    order_override: Optional[List[int]] = None
    last_gathered: Optional[torch.Tensor] = None   # CPU backend: last gathered A (skip_comm)

    @property
    def max_chunks(self) -> int:
        """Ticket words per source: one per 128 rows of the largest shard (the granularity of a
        call's tickets is chosen per call, see ``_ticket_rows``)."""
        return max(1, (self.max_M // self.num_ranks) // 128)

    @property
    def ws_ptr(self) -> int:
        return self.ws.local_ptr

    def workspace(self, parity: int, M: int) -> torch.Tensor:
        """This rank's gathered A of the given parity as a [M, K] tensor."""
        off = parity * self.max_M * self.K * 2
        return self.ws.tensor(self.input_dtype, (M, self.K), off, rank=self.rank)


def create_ag_gemm_intra_node_context(max_M, K, input_dtype, output_dtype, rank, num_ranks, mpi=None,
                                      comm=None, M_PER_CHUNK=1024, ag_stream=None, gemm_stream=None,
                                      world=None, transport: Optional[str] = None):
    """Collective. Allocates the symmetric workspace and ticket planes.

    ``mpi`` is accepted for signature compatibility and ignored; ``comm`` may be
    a ``torch.distributed`` process group. ``transport``: see the module docstring.
    """
    assert max_M % num_ranks == 0, "max_M must be divisible by num_ranks"
    m_pr = max_M // num_ranks
    M_PER_CHUNK = min(M_PER_CHUNK, m_pr)
    assert m_pr % M_PER_CHUNK == 0, "rows per rank must be a multiple of M_PER_CHUNK"
    assert M_PER_CHUNK % 128 == 0, "M_PER_CHUNK must be a multiple of 128"
    if world is None:
        world = default_world() or init_runtime(rank, num_ranks, comm)
    ctx = AllGatherGEMMTensorParallelContext(rank=rank, num_ranks=num_ranks, max_M=max_M, K=K,
                                             input_dtype=input_dtype, output_dtype=output_dtype,
                                             M_PER_CHUNK=M_PER_CHUNK, world=world,
                                             ag_stream=ag_stream, gemm_stream=gemm_stream)
    if isinstance(world, CpuWorld):
        return ctx
    assert input_dtype == output_dtype, "the fused kernel emits the input dtype"
    want = transport or env_str("TRIDIST_AG_TRANSPORT", "auto")
    assert want in ("auto", "mc", "push", "pull")
    ws_bytes = 2 * max_M * K * 2
    # "auto" is the bulk-copy push: measured against the multicast form it is equal at 4 GPUs and 12 %
    # faster at 8 (every GPU then receives eight multicast streams at once, more than its links take)
    if num_ranks > 1 and want == "mc" and env_int("TRIDIST_NVLS", 1):
        ctx.mc = world.alloc_multicast(ws_bytes)
    if want == "mc" and ctx.mc is None:
        raise RuntimeError("tridist_b200: transport 'mc' needs a multicast-bound workspace: "
                           + str(getattr(world, "multicast_unavailable", "not a multi-process world")))
    ctx.ws = ctx.mc if ctx.mc is not None else world.alloc(ws_bytes, rank)
    ctx.transport = "mc" if ctx.mc is not None else ("pull" if want == "pull" else "push")
    ctx.flags = world.alloc(num_ranks * ctx.max_chunks * 4, rank)
    ctx.arrive = world.alloc(num_ranks * ctx.max_chunks * 4, rank)
    ctx.counters = torch.zeros((num_ranks + 1) * ctx.max_chunks, dtype=torch.int32, device="cuda")
    ctx.arrival_ns = torch.zeros(num_ranks, dtype=torch.int64, device="cuda")
    if ctx.mc is not None and env_int("TRIDIST_NVLS_SELFTEST", 1):
        _mc_selftest(ctx)
    world.host_barrier()
    return ctx


def _mc_selftest(ctx) -> None:
    """Collective. Two small all-gathers of known integers through the multicast workspace (both
    parities); if any rank sees a wrong value or a kernel-reported failure, all ranks drop the
    multicast workspace together and the context falls back to the bulk-copy push."""
    import torch.distributed as dist
    world, R, rank = ctx.world, ctx.num_ranks, ctx.rank
    m_pr = min(ctx.max_M // R, 128)
    dev = torch.device("cuda", world.device)
    a = torch.full((m_pr, ctx.K), float(rank + 1), dtype=ctx.input_dtype, device=dev)
    b = torch.zeros((128, ctx.K), dtype=ctx.input_dtype, device=dev)
    b[:, :64] = 1.0
    why = ""
    try:
        for _ in range(2):
            c = torch.empty((m_pr * R, 128), dtype=ctx.output_dtype, device=dev)
            ag_gemm_intra_node_op(a, b, c, ctx)
            torch.cuda.synchronize()
            world.check()
            expect = (torch.arange(R, device=dev).repeat_interleave(m_pr).float() + 1.0) * 64.0
            bad = int((c.float() != expect[:, None]).sum().item())
            if bad:
                why = f"{bad} of {c.numel()} values differ"
                break
    except Exception as exc:
        why = f"{type(exc).__name__}: {exc}"
        try:
            world.clear_status()
        except Exception:
            pass
    ctx.plans.clear()
    verdicts = [None] * R
    dist.all_gather_object(verdicts, why, group=world.group)
    if any(verdicts):
        world.multicast_unavailable = "all-gather self-test failed: " + "; ".join(
            f"rank {r}: {v}" for r, v in enumerate(verdicts) if v)
        world.free_multicast(ctx.mc)
        ctx.mc = None
        ctx.ws = world.alloc(2 * ctx.max_M * ctx.K * 2, rank)
        ctx.transport = "push"
        ctx.flag_round = 0
        for buf in (ctx.flags, ctx.arrive):
            native().fill_u32(buf.local_ptr, buf.nbytes // 4, 0)
        torch.cuda.synchronize()


def _ticket_rows(ctx, m_pr: int) -> int:
    """Rows per arrival ticket: ``M_PER_CHUNK`` of the context, cut down to ``TRIDIST_AG_TICKET_ROWS``
    (default 256, the rows of one CTA tile) so that a consumer can start on a shard as soon as its
    first rows have landed instead of waiting for all of it."""
    rows = min(ctx.M_PER_CHUNK, m_pr)
    want = env_int("TRIDIST_AG_TICKET_ROWS", 256)
    if want >= 128 and want % 128 == 0 and want < rows and rows % want == 0 and m_pr // want <= 32:
        rows = want
    return rows


def _push_parts(chunk_rows: int, K: int) -> int:
    """Pieces of work a chunk's push is cut into (whole rows each, about a megabyte)."""
    parts = 1
    while parts < 64 and chunk_rows % (parts * 2) == 0 and (chunk_rows // (parts * 2)) * K * 2 >= (1 << 20):
        parts *= 2
    return parts


def _push_plan(M: int, N_out: int, K: int, m_pr: int, R: int, bn_out: int, want_ctas: int = 0,
               multicast: bool = False):
    """(pushing CTAs, scheduling rounds they sit out). The pushing CTAs carry the whole shard to
    the peers before they compute anything; they skip as many rounds of tiles as that takes.
    ``multicast``: the shard leaves once, as multimem stores by the CTAs' communication warps."""
    m_tiles = M // BM
    wide = env_int("TRIDIST_WIDE", 1) and m_tiles >= 4 and (m_pr // BM) % 4 == 0
    pair = env_int("TRIDIST_CTA_PAIR", 1) and (m_pr // BM) % 2 == 0
    unit_rows = 512 if (wide and pair) else (256 if pair else 128)
    workers = 148 // (2 if pair else 1)
    units = ((M + unit_rows - 1) // unit_rows) * ((N_out + bn_out - 1) // bn_out)
    rounds = units / float(workers)
    tile_us = unit_rows * 256.0 * 2.0 * K / ((2 if pair else 1) * 8192.0 * 1500.0)
    out_bytes = (1 if multicast else R - 1) * m_pr * K * 2.0
    # measured: about 34 GB/s per CTA of the bulk-copy push (twelve 16 KB pieces in flight), 560 GB/s at
    # most; multimem stores (128 threads, eight 16-byte pieces each): 8, 16 and 24 CTAs all send 50 MB in
    # 0.48-0.51 ms at 4 GPUs, so at least 13 GB/s per CTA and about 105 GB/s per GPU at most
    per_cta, cap, max_ctas = (13.0, 105.0, 16) if multicast else (34.0, 560.0, 32)
    forced_ctas, forced_skip = env_int("TRIDIST_PUSH_CTAS", -1), env_int("TRIDIST_PUSH_SKIP", -1)
    if forced_ctas < 0 and want_ctas > 0:
        forced_ctas = want_ctas

    def push_us(ctas: int) -> float:
        return out_bytes / (min(ctas * per_cta, cap) * 1e3)

    def skip_of(ctas: int) -> int:
        return max(0, min(int(math.ceil(push_us(ctas) / tile_us)), max(int(rounds) - 1, 0)))

    if forced_ctas >= 0:
        ctas = forced_ctas
    else:
        # fewest CTA-rounds given up to the push, among the counts that finish it by 60 % of the kernel
        step = 2 if pair else 1
        best = None
        for n in range(4, max_ctas + 1, step):
            if push_us(n) > 0.6 * rounds * tile_us and n < max_ctas:
                continue
            cost = n * skip_of(n)
            if best is None or cost < best[0]:
                best = (cost, n)
        ctas = best[1] if best else 16
    skip = forced_skip if forced_skip >= 0 else skip_of(ctas if ctas > 0 else 148)
    return ctas, skip


def _plan(ctx, a, b, c, swiglu=False):
    R, rank = ctx.num_ranks, ctx.rank
    m_pr, K = a.shape
    M = m_pr * R
    n_rows = b.shape[0]
    N = n_rows // 2 if swiglu else n_rows
    bn = choose_bn(M, N, swiglu, K=K)
    order = ctx.order_override or rotation_order(rank, R, 1, own_last=False)
    # emulated launches cannot take a per-call table: a device order table is baked into the plan
    baked_table = getattr(ctx, "emu_order_table", None)
    key = (a.data_ptr(), b.data_ptr(), c.data_ptr(), m_pr, n_rows, K, a.stride(0), b.stride(0), c.stride(0),
           a.dtype, swiglu, bn, tuple(order), baked_table.data_ptr() if baked_table is not None else 0,
           ctx.observe, getattr(ctx, "emu_table_header", False), getattr(ctx, "seg_bands", 0), getattr(ctx, "seg_own_first", 0), ctx.transport,
           ctx.push_ctas)

    def make():
        d = base_desc(ctx.world, rank, R, a, b, c.data_ptr(), c.stride(0), M, N, K, bn, OP_AG)
        d["a_rows"] = m_pr
        d["m_per_rank"] = m_pr
        d["sched"] = SCHED_SEGMENT if (m_pr % BM == 0) else SCHED_NATURAL
        d["seg_order"] = order
        if baked_table is not None:
            d["order_table"] = baked_table.data_ptr()
            d["order_table_header"] = 1 if getattr(ctx, "emu_table_header", False) else 0
        d["seg_bands"] = int(getattr(ctx, "seg_bands", 0) or 0)
        d["seg_own_first"] = int(getattr(ctx, "seg_own_first", 0) or 0)
        if swiglu:
            d["epi"] = EPI_SWIGLU
            d["swiglu_up_row0"] = N
        if R > 1:
            half = ctx.max_M * K * 2
            d["peer_ws"] = [ctx.ws.ptrs(0), ctx.ws.ptrs(half)]
            d["peer_ag_flags"] = ctx.flags.ptrs()
            d["ag_flag_stride"] = ctx.max_chunks     # one word per (source, chunk) for every M
            d["ag_counters"] = ctx.counters.data_ptr()
            d["arrival_ns"] = ctx.arrival_ns.data_ptr() if ctx.observe else 0
            chunk = _ticket_rows(ctx, m_pr)
            d["chunk_rows"] = chunk
            d["n_chunks"] = m_pr // chunk
            d["push_parts"] = _push_parts(chunk, K)
            # A subset of the CTAs carries the push (their operand ring is the copy ring
            # meanwhile) and joins the GEMM as many rounds late as the push takes.
            if ctx.transport == "mc":
                d["nvls"] = 1
                d["mc_part"] = [ctx.mc.mc_ptr, ctx.mc.mc_ptr + half]
                d["push_ctas"], d["push_skip_rounds"] = _push_plan(M, N, K, m_pr, R, bn // 2 if swiglu else bn,
                                                                   ctx.push_ctas, multicast=True)
                if not d["seg_bands"] and baked_table is None and ctx.order_override is None:
                    # every source's rows arrive at the same rate: own rows first, then the first
                    # row unit of every source, then the second ...
                    d["seg_bands"], d["seg_own_first"] = -1, 1
            else:
                d["push_ctas"], d["push_skip_rounds"] = _push_plan(M, N, K, m_pr, R, bn // 2 if swiglu else bn,
                                                                   ctx.push_ctas)
            if ctx.transport == "pull":
                d["ag_pull"] = 1
                d["peer_ag_arrive"] = ctx.arrive.ptrs()
            debug_check(d, c_bytes=tensor_extent_bytes(c), ws_bytes=ctx.max_M * K * 2,
                        ag_flag_words=ctx.flags.nbytes // 4)
        else:
            debug_check(d, c_bytes=tensor_extent_bytes(c))
        return native().gemm_plan_create(d)

    return ctx.plans.get(key, make)


def _check_args(a, b, c, ctx):
    m_pr, K = a.shape
    M = m_pr * ctx.num_ranks
    assert K == ctx.K and M <= ctx.max_M, "shape exceeds the context"
    assert a.dtype == ctx.input_dtype and b.dtype == ctx.input_dtype
    assert a.stride(1) == 1 and b.stride(1) == 1 and a.stride(0) == K, "a must be a contiguous [M_pr, K] shard"
    assert M % _CONSUMER_BLOCK_M == 0 and b.shape[0] % _CONSUMER_BLOCK_N == 0
    assert K % 16 == 0
    assert m_pr % min(ctx.M_PER_CHUNK, m_pr) == 0
    assert c.shape[0] == M and c.stride(1) == 1


def ag_gemm_intra_node_op(a, b, c, ctx, skip_comm=False, order_table: Optional[torch.Tensor] = None,
                          fuse_swiglu: bool = False, comm_only: bool = False, table_header: bool = False):
    """``c[M, N_pr] = allgather_M(a) @ b.T``.

    ``skip_comm=True`` is the GEMM-only decomposition mode: the kernel multiplies
    the workspace left by the last full call and pushes nothing.
    ``order_table`` (device int32[R]) overrides the source visiting order for this
    call (skew-aware scheduling); with ``table_header=True`` it is the ``order[]`` part of a full
    skew table ``[seq, degraded, mode, k_eff, order[R], budget[R]]`` and the kernel also honours
    the mode (band-major / source-major walk), ``k_eff`` (row bands), ``degraded`` and the
    per-source spin budgets. ``fuse_swiglu`` treats b as ``[gate; up]`` and
    writes ``silu(gate) * up`` (c has N_pr/2 columns). ``comm_only=True`` is the push-only
    decomposition mode: the shard is pushed and the tickets are raised, no tile is computed.
    """
    if isinstance(ctx.world, CpuWorld):
        return cpu_backend.ag_gemm(a, b, c, ctx, skip_comm, fuse_swiglu)
    _check_args(a, b, c, ctx)
    if not skip_comm:
        ctx.flag_round = next_round(ctx.flag_round, "all-gather context")
    if ctx.flag_round == 0:
        raise RuntimeError("skip_comm=True needs a full call on this context first")
    if ctx.observe and not skip_comm:
        ctx.arrival_ns.fill_(torch.iinfo(torch.int64).max)
    pid = _plan(ctx, a, b, c, fuse_swiglu)
    native().gemm_plan_launch(pid, ctx.flag_round, ctx.flag_round & 1,
                              order_table.data_ptr() if order_table is not None else 0,
                              (1 if skip_comm else 0) | (2 if comm_only else 0) |
                              (8 if (table_header and order_table is not None) else 0))
    return c


def ag_gemm_intra_node(a, b, transe_b, ctx):
    """Allocating wrapper (reference signature; ``transe_b=True`` is not supported there either)."""
    if transe_b:
        raise NotImplementedError("transe_b=True is not implemented")
    M = a.shape[0] * ctx.num_ranks
    c = torch.empty((M, b.shape[0]), dtype=ctx.output_dtype, device=a.device)
    return ag_gemm_intra_node_op(a, b, c, ctx)


def ag_gemm_emulated(ctxs, a_list, b_list, c_list, skip_comm=False, fuse_swiglu=False, mute_ranks=()):
    """All ranks of an ``EmulatedWorld`` in one cooperative launch (single-GPU protocol test).
    ``mute_ranks``: virtual ranks that neither push nor wait in this call; the others wait for
    their shards in vain, the bounded wait runs out and the kernel reports it (the give-up path)."""
    for ctx, a, b, c in zip(ctxs, a_list, b_list, c_list):
        _check_args(a, b, c, ctx)
        if not skip_comm:
            ctx.flag_round = next_round(ctx.flag_round, "all-gather context")
    pids = [_plan(ctx, a, b, c, fuse_swiglu) for ctx, a, b, c in zip(ctxs, a_list, b_list, c_list)]
    rnd = ctxs[0].flag_round
    flags = (1 if skip_comm else 0) | sum(1 << (8 + int(r)) for r in mute_ranks)
    native().gemm_plans_launch_emulated(pids, rnd, rnd & 1, flags)
    return c_list


def finalize_ag_gemm_context(ctx) -> None:
    """Collective: release the symmetric buffers of the context."""
    if ctx.ws is None:
        return
    ctx.plans.clear()
    if not isinstance(ctx.world, EmulatedWorld):
        if ctx.mc is not None:
            ctx.world.free_multicast(ctx.mc)
            ctx.mc = None
        else:
            ctx.world.free(ctx.ws)
        ctx.world.free(ctx.flags)
        if ctx.arrive is not None:
            ctx.world.free(ctx.arrive)
    ctx.ws = ctx.flags = ctx.arrive = None
