"""GEMM+AR by recursive doubling over row panels (reference: triton_dist/kernels/dcu/gemm_ar_rd.py:268-522).

``C = sum_r a_r @ b_r.T`` with the full C on every rank, log2(R) pairwise panel exchanges
instead of a full-mesh fan-out, and no global barrier inside the op:

* the rows of C are cut into panels of ``chunk_rows`` rows (about ``target_chunks`` panels, not
  below ``min_chunk_rows``, as the reference derives them at gemm_ar_rd.py:317-329);
* per panel the tcgen05 GEMM writes this rank's partial straight into ``c`` (the accumulator of
  the exchange), on the caller's stream and on all SMs but the few kept for the exchange;
* per panel one exchange kernel (``csrc/ops/rd_exchange.cu``) runs on the context's side stream:
  for phase p it pushes its slice of the accumulator into the staging slot of partner
  ``rank ^ (1 << p)``, raises the partner's arrival ticket, waits (bounded) for the partner's,
  adds the partner's snapshot in place and acks; the GEMM of panel i + 1 overlaps the
  exchange of panel i;
* ``stage_slots`` staging slots are recycled under monotonic arrival / ack tickets
  (``ticket = round_base + panel + 1``; ``round_base`` advances by ``num_chunks + 1`` per call, so
  calls with different M never collide), bounded by ``MAX_TICKETS``.

Both partners add the same two 16-bit panels in fp32 and round once, so all ranks hold
bit-identical results after the last phase.

On NVSwitch the fused two-shot / switch-reduced kernel of ``gemm_allreduce`` moves fewer bytes per
rank and is the faster all-reduce; ``TRIDIST_RD_TRANSPORT=mesh`` (or ``transport="mesh"``) makes
these entry points use it. ``wait_mode`` ("stream" | "spin" in the reference: a stream memory wait
or a one-CTA spin kernel) has one form here, the bounded in-kernel wait, because a stream
memory wait has no limit; a non-default value is reported once and ignored.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..parallel.runtime import CpuWorld, EmulatedWorld, SymmBuffer, native
from ..utils.config import env_int, env_str
from ._gemm_common import gemm_nt, warn_ignored
from .gemm_allreduce import (GemmARContext, create_gemm_ar_intra_node_context, finalize_gemm_ar_context,
                             gemm_ar_intra_node, gemm_ar_intra_node_op)

GemmARRDContext = GemmARContext
MAX_TICKETS = 1 << 20
PANEL_BYTES_CAP = 8 << 20      # a panel push stays below 8 MB at large N
RD_MAX_SLICES = 64             # ticket row length (kRdMaxSlices of the kernel)


@dataclass
class RdState:
    """What the recursive-doubling transport adds to an all-reduce context."""
    chunk_rows: int
    num_chunks: int
    stage_slots: int
    phases: int
    slot_bytes: int
    comm_ctas: int
    transport: str
    scatter: Optional[SymmBuffer] = None      # [slots][phases][chunk_rows * N] 16-bit
    arrival: Optional[SymmBuffer] = None      # u32 [slots][phases][RD_MAX_SLICES]
    ack: Optional[SymmBuffer] = None          # same shape
    round_base: int = 0
    round_stride: int = 0
    last_ticket_per_slot: List[int] = field(default_factory=list)
    side_stream: Optional[torch.cuda.Stream] = None


def panel_rows(max_M: int, N: int, chunk_rows: int = 0, target_chunks: int = 4, min_chunk_rows: int = 512,
               elem_bytes: int = 2) -> int:
    """Rows of one panel: the caller's ``chunk_rows``, or about ``target_chunks`` panels, at least
    ``min_chunk_rows`` rows, 256-row aligned, and at most 8 MB of panel (gemm_ar_rd.py:317-329 there)."""
    if chunk_rows and chunk_rows > 0:
        return max(64, min(int(chunk_rows), max_M) // 64 * 64)
    rows = -(-max_M // max(1, target_chunks))
    rows = min(max(rows, min_chunk_rows), max_M)
    rows = min(-(-rows // 256) * 256, max_M)
    cap = max(256, -(-(PANEL_BYTES_CAP // max(1, N * elem_bytes)) // 256) * 256)
    return max(64, min(rows, cap) // 64 * 64)


def partners_of(rank: int, num_ranks: int) -> List[int]:
    return [rank ^ (1 << p) for p in range(num_ranks.bit_length() - 1)]


def create_gemm_ar_rd_context(max_M, N, input_dtype, output_dtype, rank, num_ranks, mpi=None, comm=None,
                              chunk_rows=0, target_chunks=4, min_chunk_rows=512, stage_slots=4,
                              wait_mode=None, world=None, transport: Optional[str] = None):
    """Collective. The all-reduce context plus the staging slots and the two ticket planes of the
    panel exchange on the symmetric heap."""
    assert num_ranks & (num_ranks - 1) == 0, "recursive doubling needs 2^k ranks"
    assert input_dtype == output_dtype, "panels are exchanged in output dtype"
    assert N % 128 == 0 and max_M % 64 == 0
    ctx = create_gemm_ar_intra_node_context(max_M, N, input_dtype, output_dtype, rank, num_ranks, mpi, comm,
                                            M_PER_CHUNK=64, world=world)
    rows = panel_rows(max_M, N, chunk_rows, target_chunks, min_chunk_rows)
    ctx.chunk_rows = rows
    num_chunks = -(-max_M // rows)
    slots = max(1, min(int(stage_slots), num_chunks))
    phases = num_ranks.bit_length() - 1
    rd = RdState(chunk_rows=rows, num_chunks=num_chunks, stage_slots=slots, phases=phases,
                 slot_bytes=rows * N * 2, comm_ctas=max(1, min(RD_MAX_SLICES, env_int("TRIDIST_RD_CTAS", 16))),
                 transport=transport or env_str("TRIDIST_RD_TRANSPORT", "rd"),
                 round_stride=num_chunks + 1, last_ticket_per_slot=[0] * slots)
    assert rd.transport in ("rd", "mesh")
    ctx.rd = rd
    warn_ignored("create_gemm_ar_rd_context", wait_mode=(wait_mode, None))
    w = ctx.world
    if isinstance(w, CpuWorld) or num_ranks == 1 or rd.transport == "mesh":
        return ctx
    rd.scatter = w.alloc(slots * phases * rd.slot_bytes, rank)
    rd.arrival = w.alloc(slots * phases * RD_MAX_SLICES * 4, rank)
    rd.ack = w.alloc(slots * phases * RD_MAX_SLICES * 4, rank)
    if not isinstance(w, EmulatedWorld):
        rd.side_stream = torch.cuda.Stream(device=w.device)
    w.host_barrier()
    return ctx


def _rank_args(ctx, c_panel, rows: int, slot: int, ticket: int, prev: int) -> dict:
    rd, w, rank = ctx.rd, ctx.world, ctx.rank
    partners = partners_of(rank, ctx.num_ranks)
    return dict(c=c_panel.data_ptr(), ldc=c_panel.stride(0), rows=rows, n_cols=ctx.N, phases=rd.phases,
                slot=slot, slots=rd.stage_slots, flag_slices=RD_MAX_SLICES, slot_bytes=rd.slot_bytes,
                scatter=rd.scatter.peer_ptrs[rank], peer_scatter=[rd.scatter.peer_ptrs[q] for q in partners],
                arrival=rd.arrival.peer_ptrs[rank], ack=rd.ack.peer_ptrs[rank],
                peer_arrival=[rd.arrival.peer_ptrs[q] for q in partners],
                peer_ack=[rd.ack.peer_ptrs[q] for q in partners],
                ticket=ticket, prev_ticket=prev, rank=rank, status_dev=w.status_dev,
                abort_word=w.abort_word_of(rank), timeout_ns=w.timeout_ns, peer_abort=w.peer_abort_words())


def _check(a, b, c, ctx):
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K and tuple(c.shape) == (M, N) and N == ctx.N
    assert M <= ctx.max_M and M % 64 == 0 and K % 16 == 0
    assert a.dtype == ctx.input_dtype and b.dtype == ctx.input_dtype and c.dtype == ctx.output_dtype
    assert c.stride(1) == 1 and c.stride(0) % 8 == 0
    return M, N, K


def _advance(ctx, n_tasks: int) -> int:
    rd = ctx.rd
    rd.round_base += rd.round_stride
    if rd.round_base + n_tasks >= MAX_TICKETS:
        raise RuntimeError("tridist_b200: recursive-doubling context ran out of tickets "
                           f"({MAX_TICKETS}); create a new context")
    return rd.round_base


def _gemm_ctas(ctx) -> int:
    sms = torch.cuda.get_device_properties(ctx.world.device).multi_processor_count
    return max(2, (sms - ctx.rd.comm_ctas) // 2 * 2)


def gemm_ar_rd_op(a, b, c, ctx, component="full"):
    """``c = sum_r a_r @ b_r.T`` on every rank through the panel pipeline. Everything is enqueued
    up front; the exchange kernels pace themselves on tickets. ``component="gemm"``: the panel GEMMs
    only (decomposition; tickets are not advanced)."""
    rd = getattr(ctx, "rd", None)
    assert component in ("full", "gemm")
    if rd is None or isinstance(ctx.world, CpuWorld) or ctx.num_ranks == 1 or rd.transport == "mesh":
        return gemm_ar_intra_node_op(a, b, c, ctx, component=component)
    M, N, K = _check(a, b, c, ctx)
    CR, S = rd.chunk_rows, rd.stage_slots
    n_tasks = -(-M // CR)
    full = component == "full"
    base = _advance(ctx, n_tasks) if full else 0
    main = torch.cuda.current_stream()
    side = rd.side_stream
    bf16 = ctx.output_dtype == torch.bfloat16
    max_ctas = _gemm_ctas(ctx) if full else 0
    for i in range(n_tasks):
        r0 = i * CR
        rows = min(CR, M - r0)
        c_panel = c[r0:r0 + rows]
        gemm_nt(a[r0:r0 + rows], b, out=c_panel, max_ctas=max_ctas)
        if not full:
            continue
        slot = i % S
        ticket = base + i + 1
        prev, rd.last_ticket_per_slot[slot] = rd.last_ticket_per_slot[slot], ticket
        ev = torch.cuda.Event()
        ev.record(main)
        side.wait_event(ev)
        with torch.cuda.stream(side):
            native().rd_exchange([_rank_args(ctx, c_panel, rows, slot, ticket, prev)], rd.comm_ctas, bf16)
    if full:
        main.wait_stream(side)
    return c


def gemm_ar_rd(a, b, ctx):
    rd = getattr(ctx, "rd", None)
    if rd is None or isinstance(ctx.world, CpuWorld) or ctx.num_ranks == 1 or rd.transport == "mesh":
        return gemm_ar_intra_node(a, b, ctx)
    c = torch.empty((a.shape[0], b.shape[0]), dtype=ctx.output_dtype, device=a.device)
    return gemm_ar_rd_op(a, b, c, ctx)


def gemm_ar_rd_emulated(ctxs, a_list, b_list, c_list):
    """All virtual ranks of an ``EmulatedWorld`` in one process: per panel the R panel GEMMs, then ONE
    cooperative launch of the exchange kernel over all ranks (kernels that wait on one another
    never run as separate launches on one GPU)."""
    R = len(ctxs)
    M, N, K = _check(a_list[0], b_list[0], c_list[0], ctxs[0])
    rd0 = ctxs[0].rd
    CR, S = rd0.chunk_rows, rd0.stage_slots
    n_tasks = -(-M // CR)
    bases = [_advance(ctx, n_tasks) for ctx in ctxs]
    bf16 = ctxs[0].output_dtype == torch.bfloat16
    for i in range(n_tasks):
        r0 = i * CR
        rows = min(CR, M - r0)
        blocks = []
        for ctx, a, b, c, base in zip(ctxs, a_list, b_list, c_list, bases):
            c_panel = c[r0:r0 + rows]
            gemm_nt(a[r0:r0 + rows], b, out=c_panel)
            slot = i % S
            ticket = base + i + 1
            prev, ctx.rd.last_ticket_per_slot[slot] = ctx.rd.last_ticket_per_slot[slot], ticket
            blocks.append(_rank_args(ctx, c_panel, rows, slot, ticket, prev))
        native().rd_exchange(blocks, min(rd0.comm_ctas, 16), bf16)
    return c_list


def finalize_gemm_ar_rd_context(ctx):
    rd = getattr(ctx, "rd", None)
    if rd is not None and rd.scatter is not None and not isinstance(ctx.world, EmulatedWorld):
        for buf in (rd.scatter, rd.arrival, rd.ack):
            ctx.world.free(buf)
    if rd is not None:
        rd.scatter = rd.arrival = rd.ack = None
    finalize_gemm_ar_context(ctx)
