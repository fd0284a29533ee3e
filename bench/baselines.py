"""cuBLAS + NCCL serial baselines: the bar every fused operator has to beat.

Same recipe as the reference's 8-card bench (bench/s9_bench_8card.py:150-358 and
bench/s21_bench_tp_mlp_dcu.py:209-219): the vendor GEMM (``torch.matmul``) run back
to back with the library collective on one stream —
  AG+GEMM   all_gather_into_tensor -> matmul
  GEMM+RS   matmul -> reduce_scatter_tensor
  GEMM+AR   matmul -> all_reduce
  MoE       all_to_all_single x2 with equal, padded splits
None of this library's kernels is on these paths.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F


class AGGemmBaseline:
    def __init__(self, m_pr, K, n_loc, R, dtype, group=None):
        self.R, self.group = R, group
        self.full = torch.empty((m_pr * R, K), dtype=dtype, device="cuda")
        self.c = torch.empty((m_pr * R, n_loc), dtype=dtype, device="cuda")

    def __call__(self, a, b):
        if self.R > 1:
            dist.all_gather_into_tensor(self.full, a, group=self.group)
            torch.matmul(self.full, b.t(), out=self.c)
        else:
            torch.matmul(a, b.t(), out=self.c)
        return self.c


class GemmRSBaseline:
    def __init__(self, M, N, R, dtype, group=None):
        self.R, self.group = R, group
        self.partial = torch.empty((M, N), dtype=dtype, device="cuda")
        self.out = torch.empty((M // R, N), dtype=dtype, device="cuda")

    def __call__(self, a, b):
        torch.matmul(a, b.t(), out=self.partial)
        if self.R > 1:
            dist.reduce_scatter_tensor(self.out, self.partial, group=self.group)
            return self.out
        return self.partial


class GemmARBaseline:
    def __init__(self, M, N, R, dtype, group=None):
        self.R, self.group = R, group
        self.c = torch.empty((M, N), dtype=dtype, device="cuda")

    def __call__(self, a, b):
        torch.matmul(a, b.t(), out=self.c)
        if self.R > 1:
            dist.all_reduce(self.c, group=self.group)
        return self.c


class MoEBaseline:
    """all_to_all_single for dispatch and again for combine, carrying exactly the rows the
    routing sends between each pair of ranks (uneven splits). The reference's bench uses equal
    padded splits (bench/s9_bench_8card.py:332-340); exact splits move fewer bytes and are the
    stronger baseline, and they stay meaningful under skewed routing."""

    def __init__(self, idx, E, H, R, dtype, group=None):
        self.R, self.group = R, group
        epr = E // R
        dest = (idx.long() // epr).flatten()
        send = torch.bincount(dest, minlength=R).to(torch.int64)            # rows I send to each rank
        if R > 1:
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=group)
        else:
            recv = send.clone()
        self.send_splits = send.cpu().tolist()
        self.recv_splits = recv.cpu().tolist()
        rank = dist.get_rank(group) if R > 1 else 0
        mine_in = sum(v for i, v in enumerate(self.recv_splits) if i != rank)
        mine_out = sum(v for i, v in enumerate(self.send_splits) if i != rank)
        if R > 1:
            t = torch.tensor([mine_in, mine_out], dtype=torch.int64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            mine_in, mine_out = int(t[0]), int(t[1])
        self.recv_splits_remote_rows, self.send_splits_remote_rows = mine_in, mine_out
        self.send = torch.empty((sum(self.send_splits), H), dtype=dtype, device="cuda")
        self.recv = torch.empty((sum(self.recv_splits), H), dtype=dtype, device="cuda")
        self.back = torch.empty_like(self.send)

    def __call__(self):
        if self.R > 1:
            dist.all_to_all_single(self.recv, self.send, self.recv_splits, self.send_splits, group=self.group)
            dist.all_to_all_single(self.back, self.recv, self.send_splits, self.recv_splits, group=self.group)
        else:
            self.recv.copy_(self.send)
            self.back.copy_(self.recv)
        return self.back


class TPMLPBaseline:
    """AG -> matmul -> silu*up -> matmul -> RS with torch ops only."""

    def __init__(self, M, K, i_loc, R, dtype, group=None):
        self.R, self.group, self.i_loc = R, group, i_loc
        self.x_full = torch.empty((M, K), dtype=dtype, device="cuda")
        self.h = torch.empty((M, 2 * i_loc), dtype=dtype, device="cuda")
        self.partial = torch.empty((M, K), dtype=dtype, device="cuda")
        self.y = torch.empty((M // R, K), dtype=dtype, device="cuda")

    def __call__(self, x_loc, w_gu, w_down):
        if self.R > 1:
            dist.all_gather_into_tensor(self.x_full, x_loc, group=self.group)
            x = self.x_full
        else:
            x = x_loc
        torch.matmul(x, w_gu.t(), out=self.h)
        h2 = F.silu(self.h[:, :self.i_loc]) * self.h[:, self.i_loc:]
        torch.matmul(h2, w_down.t(), out=self.partial)
        if self.R > 1:
            dist.reduce_scatter_tensor(self.y, self.partial, group=self.group)
            return self.y
        return self.partial
