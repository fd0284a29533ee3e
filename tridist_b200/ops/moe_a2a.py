"""MoE all-to-all: dispatch token rows to expert ranks, combine expert outputs back.

Public API follows the reference (triton_dist/kernels/dcu/moe_a2a.py:287-555):

* ``create_moe_a2a_intra_node_context(num_experts, hidden, dtype, max_tokens, topk, rank,
  num_ranks, mpi, comm, BLOCK_H=1024)``
* ``moe_dispatch_intra_node_op(tokens, topk_idx, ctx, component="full")`` -> device int32[1]
  ``recv_total``; afterwards ``ctx.recv`` holds the received rows ordered by (source rank,
  local expert) segments and ``ctx.scatter_idx[t, j]`` the destination row of each (t, j)
* the expert phase writes ``ctx.out[row]`` for ``row < recv_total``
* ``moe_combine_intra_node_op(ctx, topk_idx, output, topk_weights=None)``:
  ``output[t] = sum_j w[t, j] * out_{rank(e_j)}[scatter_idx[t, j]]`` in fp32.

Per round: three kernels (metadata, dispatch, combine), no host synchronisation
and no host-issued copy; completion of the dispatch kernel means every rank's
rows have landed.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..parallel import cpu_backend
from ._gemm_common import next_round
from ..parallel.runtime import (CpuWorld, EmulatedWorld, SymmBuffer, default_world, init_runtime,
                                native)
from ._gemm_common import is_bf16


@dataclass
class MoEA2AContext:
    rank: int
    num_ranks: int
    num_experts: int
    epr: int
    hidden: int
    topk: int
    max_tokens: int
    max_recv_rows: int
    input_dtype: torch.dtype
    row_bytes: int
    BLOCK_H: int
    world: object
    recv: Optional[torch.Tensor] = None          # [max_recv_rows, H] dispatch destination
    out: Optional[torch.Tensor] = None           # [max_recv_rows, H] expert outputs (1:1 rows)
    recv_buf: Optional[SymmBuffer] = None
    out_buf: Optional[SymmBuffer] = None
    meta_buf: Optional[SymmBuffer] = None        # int32 [2][R, E] split counts by source
    flag_buf: Optional[SymmBuffer] = None        # u32 [3][R]: meta / dispatch-done / combine-ready
    scatter_idx: Optional[torch.Tensor] = None   # [max_tokens, topk] int32
    counters: Optional[torch.Tensor] = None      # [E] int32
    splits: Optional[torch.Tensor] = None        # [E] int32
    dst_row_base: Optional[torch.Tensor] = None  # [E] int32 (== [R, epr])
    recv_seg: Optional[torch.Tensor] = None      # [R, epr] int32 first row of each segment
    recv_counts: Optional[torch.Tensor] = None   # [R, epr] int32
    recv_total_t: Optional[torch.Tensor] = None  # [1] int32
    done_counter: Optional[torch.Tensor] = None
    meta_round: int = 0
    splits_all: Optional[torch.Tensor] = None    # CPU backend only

    @property
    def recv_ptr(self) -> int:
        return self.recv.data_ptr()

    @property
    def out_ptr(self) -> int:
        return self.out.data_ptr()


def create_moe_a2a_intra_node_context(num_experts, hidden, dtype, max_tokens, topk, rank, num_ranks,
                                      mpi=None, comm=None, BLOCK_H=1024, world=None,
                                      max_recv_rows: Optional[int] = None):
    """Collective. ``max_recv_rows`` defaults to the reference's worst case
    ``max_tokens * topk * num_ranks`` (every pair of every source to one rank)."""
    assert num_experts % num_ranks == 0
    BLOCK_H = min(BLOCK_H, hidden)
    assert hidden % BLOCK_H == 0 and hidden % 8 == 0
    if world is None:
        world = default_world() or init_runtime(rank, num_ranks, comm)
    elem = torch.empty((), dtype=dtype).element_size()
    if max_recv_rows is None:
        max_recv_rows = max_tokens * topk * num_ranks
    epr = num_experts // num_ranks
    ctx = MoEA2AContext(rank=rank, num_ranks=num_ranks, num_experts=num_experts, epr=epr, hidden=hidden,
                        topk=topk, max_tokens=max_tokens, max_recv_rows=max_recv_rows,
                        input_dtype=dtype, row_bytes=hidden * elem, BLOCK_H=BLOCK_H, world=world)
    dev = "cpu" if isinstance(world, CpuWorld) else "cuda"
    ctx.scatter_idx = torch.full((max_tokens, topk), -1, dtype=torch.int32, device=dev)
    ctx.counters = torch.zeros(num_experts, dtype=torch.int32, device=dev)
    ctx.splits = torch.zeros(num_experts, dtype=torch.int32, device=dev)
    ctx.dst_row_base = torch.zeros(num_experts, dtype=torch.int32, device=dev)
    ctx.recv_seg = torch.zeros((num_ranks, epr), dtype=torch.int32, device=dev)
    ctx.recv_counts = torch.zeros((num_ranks, epr), dtype=torch.int32, device=dev)
    ctx.recv_total_t = torch.zeros(1, dtype=torch.int32, device=dev)
    if isinstance(world, CpuWorld):
        ctx.recv = torch.zeros((max_recv_rows, hidden), dtype=dtype)
        ctx.out = torch.zeros((max_recv_rows, hidden), dtype=dtype)
        return ctx
    assert elem == 2, "the MoE kernels move 16-bit rows (fp16 / bf16)"
    ctx.done_counter = torch.zeros(1, dtype=torch.int32, device=dev)
    ctx.recv_buf = world.alloc(max_recv_rows * ctx.row_bytes, rank)
    ctx.out_buf = world.alloc(max_recv_rows * ctx.row_bytes, rank)
    ctx.meta_buf = world.alloc(2 * num_ranks * num_experts * 4, rank)
    ctx.flag_buf = world.alloc(3 * 64, rank)
    ctx.recv = ctx.recv_buf.tensor(dtype, (max_recv_rows, hidden), rank=rank)
    ctx.out = ctx.out_buf.tensor(dtype, (max_recv_rows, hidden), rank=rank)
    # first touch of every peer mapping (the reference's k_touch warm-up, moe_a2a.py:71, 344-347)
    for r in range(num_ranks):
        ctx.flag_buf.tensor(torch.int32, (1,), 3 * 64 - 4, rank=r).zero_()
    world.host_barrier()
    return ctx


def _desc(ctx, tokens=None, topk_idx=None, output=None, topk_weights=None, T=0):
    w = ctx.world
    par = ctx.meta_round & 1
    d = dict(rank=ctx.rank, R=ctx.num_ranks, E=ctx.num_experts, H=ctx.hidden, T=T, topk=ctx.topk,
             max_recv_rows=ctx.max_recv_rows, bf16=is_bf16(ctx.input_dtype), round=ctx.meta_round,
             tokens=tokens.data_ptr() if tokens is not None else 0,
             topk_idx=topk_idx.data_ptr() if topk_idx is not None else 0,
             topk_weights=topk_weights.data_ptr() if topk_weights is not None else 0,
             output=output.data_ptr() if output is not None else 0,
             peer_recv=ctx.recv_buf.ptrs(), peer_out=ctx.out_buf.ptrs(),
             peer_meta=ctx.meta_buf.ptrs(par * ctx.num_ranks * ctx.num_experts * 4),
             peer_meta_flags=ctx.flag_buf.ptrs(0), peer_done_flags=ctx.flag_buf.ptrs(64),
             peer_ready_flags=ctx.flag_buf.ptrs(128),
             splits=ctx.splits.data_ptr(), dst_row_base=ctx.dst_row_base.data_ptr(),
             counters=ctx.counters.data_ptr(), recv_seg=ctx.recv_seg.data_ptr(),
             recv_counts=ctx.recv_counts.data_ptr(), recv_total=ctx.recv_total_t.data_ptr(),
             scatter_idx=ctx.scatter_idx.data_ptr(), done_counter=ctx.done_counter.data_ptr(),
             status_dev=w.status_dev,
             abort_word=w.abort_word_of(ctx.rank) if hasattr(w, "abort_word_of") else w.abort_word,
             peer_abort=w.peer_abort_words() if hasattr(w, "peer_abort_words") else [],
             timeout_ns=w.timeout_ns)
    return d


def _check_dispatch(tokens, topk_idx, ctx):
    T = tokens.shape[0]
    assert T <= ctx.max_tokens, "more tokens than the context was created for"
    assert tokens.shape[1] == ctx.hidden and tokens.is_contiguous() and tokens.dtype == ctx.input_dtype
    assert topk_idx.dtype == torch.int32 and topk_idx.is_contiguous()
    assert tuple(topk_idx.shape) == (T, ctx.topk)
    return T


def moe_dispatch_intra_node_op(tokens, topk_idx, ctx, component="full"):
    """Returns the device int32[1] ``recv_total``. ``component="meta"`` stops after the
    routing metadata (split counts exchanged, segment tables built)."""
    if component not in ("full", "meta"):
        raise ValueError(f"unknown component {component!r}")
    if isinstance(ctx.world, CpuWorld):
        return cpu_backend.moe_dispatch(tokens, topk_idx, ctx, component)
    T = _check_dispatch(tokens, topk_idx, ctx)
    ctx.meta_round = next_round(ctx.meta_round, "MoE context")
    d = _desc(ctx, tokens=tokens, topk_idx=topk_idx, T=T)
    C = native()
    C.moe_meta(d)
    if component == "full":
        C.moe_dispatch(d)
    return ctx.recv_total_t


def moe_combine_intra_node_op(ctx, topk_idx, output, topk_weights=None):
    """Pull-combine of the expert outputs; must follow a dispatch of the same round."""
    if isinstance(ctx.world, CpuWorld):
        return cpu_backend.moe_combine(ctx, topk_idx, output, topk_weights)
    T = topk_idx.shape[0]
    assert output.shape[0] == T and output.shape[1] == ctx.hidden and output.is_contiguous()
    if topk_weights is not None:
        assert topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()
    d = _desc(ctx, topk_idx=topk_idx, output=output, topk_weights=topk_weights, T=T)
    native().moe_combine(d)
    return output


def moe_dispatch_emulated(ctxs: List[MoEA2AContext], tokens_list, idx_list, component="full"):
    ds = []
    for ctx, tok, idx in zip(ctxs, tokens_list, idx_list):
        T = _check_dispatch(tok, idx, ctx)
        ctx.meta_round = next_round(ctx.meta_round, "MoE context")
        ds.append(_desc(ctx, tokens=tok, topk_idx=idx, T=T))
    C = native()
    C.moe_emulated(ds, 0)
    if component == "full":
        C.moe_emulated(ds, 1)
    return [c.recv_total_t for c in ctxs]


def moe_combine_emulated(ctxs, idx_list, out_list, w_list=None):
    ds = []
    for i, (ctx, idx, out) in enumerate(zip(ctxs, idx_list, out_list)):
        w = w_list[i] if w_list is not None else None
        ds.append(_desc(ctx, topk_idx=idx, output=out, topk_weights=w, T=idx.shape[0]))
    native().moe_emulated(ds, 2)
    return out_list


def finalize_moe_a2a_context(ctx) -> None:
    if ctx.recv_buf is not None and not isinstance(ctx.world, EmulatedWorld):
        for buf in (ctx.recv_buf, ctx.out_buf, ctx.meta_buf, ctx.flag_buf):
            ctx.world.free(buf)
    ctx.recv = ctx.out = None
    ctx.recv_buf = ctx.out_buf = ctx.meta_buf = ctx.flag_buf = None
