"""CPU / gloo reference backend: the oracle for every operator family.

The reference library has no CPU path (its tests need real devices).  This
backend implements the same four API families with ``torch.distributed`` (gloo)
collectives and ``torch.matmul`` in fp32; GPU tests compare against it and the
host-side failure tests run on it.  Results are cast back to the output dtype.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist
import torch.nn.functional as F


def _world(ctx):
    return ctx.world


def _all_gather(t: torch.Tensor, world) -> List[torch.Tensor]:
    if world.num_ranks == 1:
        return [t]
    out = [torch.empty_like(t) for _ in range(world.num_ranks)]
    dist.all_gather(out, t.contiguous(), group=world.group)
    return out


def _all_reduce_sum(t: torch.Tensor, world) -> torch.Tensor:
    if world.num_ranks > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=world.group)
    return t


def _acc_dtype(dtype):
    return torch.float32 if dtype in (torch.float16, torch.bfloat16, torch.float32) else dtype


# ---------------------------------------------------------------------------
# AG + GEMM
# ---------------------------------------------------------------------------
def ag_gemm(a, b, c, ctx, skip_comm=False, fuse_swiglu=False):
    w = _world(ctx)
    if skip_comm:
        if ctx.last_gathered is None:
            raise RuntimeError("skip_comm=True needs a full call on this context first")
        full = ctx.last_gathered
    else:
        ctx.flag_round += 1
        full = torch.cat(_all_gather(a, w), dim=0)
        ctx.last_gathered = full
    acc = full.to(_acc_dtype(a.dtype)) @ b.to(_acc_dtype(b.dtype)).t()
    if fuse_swiglu:
        n = acc.shape[1] // 2
        acc = F.silu(acc[:, :n]) * acc[:, n:]
    c.copy_(acc.to(c.dtype))
    return c


# ---------------------------------------------------------------------------
# GEMM + RS / GEMM + AR
# ---------------------------------------------------------------------------
def gemm_rs(a, b, output_dtype, ctx):
    w = _world(ctx)
    partial = a.to(_acc_dtype(a.dtype)) @ b.to(_acc_dtype(b.dtype)).t()
    total = _all_reduce_sum(partial, w)
    m_pr = a.shape[0] // w.num_ranks
    return total[w.rank * m_pr:(w.rank + 1) * m_pr].to(output_dtype).contiguous()


def gemm_ar(a, b, c, ctx):
    w = _world(ctx)
    partial = a.to(_acc_dtype(a.dtype)) @ b.to(_acc_dtype(b.dtype)).t()
    total = _all_reduce_sum(partial, w)
    c.copy_(total.to(c.dtype))
    return c


# ---------------------------------------------------------------------------
# MoE all-to-all
# ---------------------------------------------------------------------------
def segment_tables(splits_all: torch.Tensor, my_rank: int, num_ranks: int, epr: int):
    """Segment algebra from the gathered split counts ``splits_all[R, E]``.

    Returns ``dst_row_base[E]`` (first row of (me, expert e) in the owner's receive
    buffer), ``recv_seg[R, epr]``, ``recv_counts[R, epr]`` and ``recv_total`` with
    the layout contract of the reference (moe_a2a.py:394-433): a destination's
    rows are ordered by (source rank, local expert).
    """
    E = splits_all.shape[1]
    s = splits_all.to(torch.int64)
    dst_row_base = torch.zeros(E, dtype=torch.int64)
    for d in range(num_ranks):
        base = int(s[:my_rank, d * epr:(d + 1) * epr].sum())
        for k in range(epr):
            dst_row_base[d * epr + k] = base
            base += int(s[my_rank, d * epr + k])
    recv_seg = torch.zeros((num_ranks, epr), dtype=torch.int64)
    recv_counts = torch.zeros((num_ranks, epr), dtype=torch.int64)
    base = 0
    for src in range(num_ranks):
        for k in range(epr):
            recv_seg[src, k] = base
            recv_counts[src, k] = s[src, my_rank * epr + k]
            base += int(recv_counts[src, k])
    return dst_row_base, recv_seg, recv_counts, int(base)


def _pad_rows(t: torch.Tensor, rows: int) -> torch.Tensor:
    out = torch.zeros((rows,) + tuple(t.shape[1:]), dtype=t.dtype)
    out[: t.shape[0]] = t
    return out


def moe_dispatch(tokens, topk_idx, ctx, component="full"):
    w = _world(ctx)
    R, E, epr = w.num_ranks, ctx.num_experts, ctx.epr
    T = tokens.shape[0]
    ctx.meta_round += 1
    idx = topk_idx.to(torch.int64)
    valid = (idx >= 0) & (idx < E)
    splits = torch.bincount(idx[valid].flatten(), minlength=E).to(torch.int32)
    splits_all = torch.stack(_all_gather(splits, w), dim=0)
    dst_row_base, recv_seg, recv_counts, recv_total = segment_tables(splits_all, w.rank, R, epr)
    ctx.splits_all = splits_all
    ctx.recv_seg.copy_(recv_seg.to(torch.int32))
    ctx.recv_counts.copy_(recv_counts.to(torch.int32))
    ctx.recv_total_t.fill_(recv_total)
    if recv_total > ctx.max_recv_rows:
        raise RuntimeError(f"receive buffer oversubscribed: {recv_total} > {ctx.max_recv_rows}")
    if component == "meta":
        return ctx.recv_total_t

    # my scatter indices: slots inside a segment follow increasing (t, j) order
    cursor = dst_row_base.clone()
    scatter = torch.full((T, ctx.topk), -1, dtype=torch.int32)
    flat = idx.flatten().tolist()
    for p, e in enumerate(flat):
        if 0 <= e < E:
            scatter[p // ctx.topk, p % ctx.topk] = int(cursor[e])
            cursor[e] += 1
    ctx.scatter_idx[:T].copy_(scatter)

    # exchange: every rank learns every rank's tokens and routing (oracle, not fast)
    tok_all = _all_gather(_pad_rows(tokens, ctx.max_tokens), w)
    idx_all = _all_gather(_pad_rows(topk_idx.to(torch.int32), ctx.max_tokens), w)
    t_all = [int(x) for x in _all_gather(torch.tensor([T], dtype=torch.int64), w)]
    cur = recv_seg.clone()
    for src in range(R):
        ids = idx_all[src][: t_all[src]].to(torch.int64).flatten().tolist()
        for p, e in enumerate(ids):
            if 0 <= e < E and e // epr == w.rank:
                k = e % epr
                ctx.recv[int(cur[src, k])] = tok_all[src][p // ctx.topk]
                cur[src, k] += 1
    return ctx.recv_total_t


def moe_combine(ctx, topk_idx, output, topk_weights=None):
    w = _world(ctx)
    epr = ctx.epr
    T = topk_idx.shape[0]
    outs = _all_gather(ctx.out, w)
    acc = torch.zeros((T, ctx.hidden), dtype=torch.float32)
    idx = topk_idx.to(torch.int64)
    for t in range(T):
        for j in range(ctx.topk):
            e = int(idx[t, j])
            row = int(ctx.scatter_idx[t, j])
            if e < 0 or e >= ctx.num_experts or row < 0:
                continue
            wgt = float(topk_weights[t, j]) if topk_weights is not None else 1.0
            acc[t] += wgt * outs[e // epr][row].to(torch.float32)
    output.copy_(acc.to(output.dtype))
    return output
