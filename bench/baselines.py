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
    """Equal-split padded all_to_all_single for dispatch and for combine; the padded
    capacity per (source, destination) pair is every pair of the source (worst case),
    as in the reference's bench (bench/s9_bench_8card.py:332-340 uses equal splits)."""

    def __init__(self, T, H, topk, R, dtype, group=None, cap_rows=None):
        self.R, self.group = R, group
        # with uniform routing a destination receives about T*topk/R rows from each source;
        # use that (rounded up by 25 %) as the fixed per-pair capacity
        cap = cap_rows or (int(T * topk / R * 1.25) + 8)
        self.cap = cap
        self.send = torch.empty((R * cap, H), dtype=dtype, device="cuda")
        self.recv = torch.empty((R * cap, H), dtype=dtype, device="cuda")
        self.back = torch.empty((R * cap, H), dtype=dtype, device="cuda")

    def __call__(self):
        if self.R > 1:
            dist.all_to_all_single(self.recv, self.send, group=self.group)
            dist.all_to_all_single(self.back, self.recv, group=self.group)
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
