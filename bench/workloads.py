"""The benchmark workloads named by BASELINE.json, as (fused, baseline, roofline) triples.

Every workload builds its inputs once (seeded, synthetic, on the CPU in pinned
memory so that the end-to-end arm can copy them in every step), creates the
fused operator's context through the public API and exposes:

  run()         the fused operator on device-resident inputs
  baseline()    the cuBLAS + NCCL composition of the same operator
  stage()       host -> device copy of this step's activations from pinned memory
  digest()      a small device tensor derived from the result (read back by the e2e arm)
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from tridist_b200.models.tp_mlp import TPMLP, TPMLPConfig
from tridist_b200.ops import (ag_gemm_intra_node_op, create_ag_gemm_intra_node_context,
                              create_gemm_ar_intra_node_context, create_gemm_rs_intra_node_context,
                              create_moe_a2a_intra_node_context, gemm_ar_intra_node,
                              gemm_rs_intra_node_op, moe_combine_intra_node_op, moe_dispatch_intra_node_op)
from tridist_b200.utils import roofline
from tridist_b200.utils.testing import moe_inputs

from . import baselines


def _pinned_randn(shape, seed, scale, dtype):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    t = (torch.randn(shape, generator=g, dtype=torch.float32) * scale).to(dtype)
    return t.pin_memory()


def _dev_randn(shape, seed, scale, dtype):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32, device="cuda") * scale).to(dtype)


def _matmul_fp32_rows(a_rows: torch.Tensor, b: torch.Tensor, chunk: int = 8192) -> torch.Tensor:
    """``a_rows.float() @ b.float().T`` without materialising b in fp32 (column chunks)."""
    af = a_rows.float()
    out = torch.empty((af.shape[0], b.shape[0]), dtype=torch.float32, device=af.device)
    for n0 in range(0, b.shape[0], chunk):
        out[:, n0:n0 + chunk] = af @ b[n0:n0 + chunk].float().t()
    return out


def _sum_over_ranks(t: torch.Tensor, R: int) -> torch.Tensor:
    if R > 1:
        dist.all_reduce(t)
    return t


def _rel_err(out: torch.Tensor, ref: torch.Tensor) -> float:
    """max |out - ref| over max |ref|: the bound of every check is relative to the result's scale."""
    return ((out.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-20)).item()


def _sample_rows(M: int, R: int, per_rank: int = 8):
    """The same rows on every rank: ``per_rank`` rows inside each rank's row block."""
    m_pr = M // R
    step = max(1, m_pr // per_rank)
    return [r * m_pr + (i * step + 3 * i) % m_pr for r in range(R) for i in range(per_rank)]


class Workload:
    """``check()`` runs the fused operator once and compares a sample of result rows with an fp32
    reference built from the same inputs (products in fp32, sums over ranks in fp32); it returns
    max |error| / max |reference| and the bench refuses to time an operator whose value exceeds
    ``tol``."""
    name: str
    h2d_bytes: int = 0
    launches_per_run: int = 1
    tol: float = 8e-3           # fp16 results, partial sums rounded to fp16 once per rank

    def run(self): ...
    def baseline(self): ...
    def stage(self): ...
    def digest(self) -> torch.Tensor: ...
    def roof(self) -> Dict: ...
    def check(self) -> float: ...


class AGGemm(Workload):
    def __init__(self, rank, R, M=8192, K=12288, N=49152, dtype=torch.float16):
        self.name = "ag_gemm"
        self.rank = rank
        self.R, self.M, self.K, self.n_loc = R, M, K, N // R
        m_pr = M // R
        s = 1.0 / math.sqrt(K)
        self.a_host = _pinned_randn((m_pr, K), 11 + rank, s, dtype)
        self.a = self.a_host.cuda()
        self.b = _dev_randn((self.n_loc, K), 101 + rank, s, dtype)
        self.c = torch.empty((M, self.n_loc), dtype=dtype, device="cuda")
        self.ctx = create_ag_gemm_intra_node_context(M, K, dtype, dtype, rank, R, M_PER_CHUNK=m_pr)
        self.base = baselines.AGGemmBaseline(m_pr, K, self.n_loc, R, dtype)
        self.h2d_bytes = self.a_host.numel() * 2

    def run(self):
        ag_gemm_intra_node_op(self.a, self.b, self.c, self.ctx)

    def baseline(self):
        return self.base(self.a, self.b)

    def stage(self):
        self.a.copy_(self.a_host, non_blocking=True)

    def digest(self):
        return self.c[0, :8].float().sum()

    def roof(self):
        return roofline.ag_gemm_roof(self.M, self.K, self.n_loc, self.R)

    def check(self):
        self.run()
        rows = _sample_rows(self.M, self.R)
        m_pr = self.M // self.R
        # the sampled rows of the gathered A: every rank contributes the rows of its own block
        mine = [(i, g - self.rank * m_pr) for i, g in enumerate(rows) if g // m_pr == self.rank]
        a_rows = torch.zeros((len(rows), self.K), dtype=torch.float32, device="cuda")
        for i, lr in mine:
            a_rows[i] = self.a[lr].float()
        _sum_over_ranks(a_rows, self.R)
        ref = _matmul_fp32_rows(a_rows, self.b)
        return _rel_err(self.c[rows], ref)


class GemmRS(Workload):
    def __init__(self, rank, R, M=8192, K=49152, N=12288, dtype=torch.float16):
        self.name = "gemm_rs"
        self.rank, self.R, self.M, self.N, self.k_loc = rank, R, M, N, K // R
        s = 1.0 / math.sqrt(K)
        self.a_host = _pinned_randn((M, self.k_loc), 21 + rank, s, dtype)
        self.a = self.a_host.cuda()
        self.b = _dev_randn((N, self.k_loc), 201 + rank, s, dtype)
        self.out = torch.empty((M // R, N), dtype=dtype, device="cuda")
        self.ctx = create_gemm_rs_intra_node_context(M, N, dtype, rank, R)
        self.base = baselines.GemmRSBaseline(M, N, R, dtype)
        self.dtype = dtype
        self.h2d_bytes = self.a_host.numel() * 2

    def run(self):
        gemm_rs_intra_node_op(self.a, self.b, self.dtype, self.rank, self.R, self.ctx, out=self.out)

    def baseline(self):
        return self.base(self.a, self.b)

    def stage(self):
        self.a.copy_(self.a_host, non_blocking=True)

    def digest(self):
        return self.out[0, :8].float().sum()

    def roof(self):
        return roofline.gemm_rs_roof(self.M, self.N, self.k_loc, self.R)

    def check(self):
        self.run()
        rows = _sample_rows(self.M, self.R)
        ref = _sum_over_ranks(_matmul_fp32_rows(self.a[rows], self.b), self.R)
        m_pr = self.M // self.R
        mine = [i for i, g in enumerate(rows) if g // m_pr == self.rank]
        return _rel_err(self.out[[rows[i] - self.rank * m_pr for i in mine]], ref[mine])


class GemmAR(Workload):
    def __init__(self, rank, R, M, K=28672, N=8192, dtype=torch.float16, mode: Optional[str] = None):
        self.name = f"gemm_ar_m{M}"
        self.R, self.M, self.N, self.k_loc = R, M, N, K // R
        s = 1.0 / math.sqrt(K)
        self.a_host = _pinned_randn((M, self.k_loc), 31 + rank + M, s, dtype)
        self.a = self.a_host.cuda()
        self.b = _dev_randn((N, self.k_loc), 301 + rank, s, dtype)
        self.ctx = create_gemm_ar_intra_node_context(M, N, dtype, dtype, rank, R, M_PER_CHUNK=64)
        if mode:
            self.ctx.mode = mode
        self.c = torch.empty((M, N), dtype=dtype, device="cuda")
        self.base = baselines.GemmARBaseline(M, N, R, dtype)
        self.h2d_bytes = self.a_host.numel() * 2

    def run(self):
        # the allocating entry point: with the two-shot algorithm it returns a view of the
        # context's symmetric result buffer, so reduced tiles land in place
        self.c = gemm_ar_intra_node(self.a, self.b, self.ctx)

    def baseline(self):
        return self.base(self.a, self.b)

    def stage(self):
        self.a.copy_(self.a_host, non_blocking=True)

    def digest(self):
        return self.c[0, :8].float().sum()

    def algorithm(self):
        """Which all-reduce form the context picks for this shape (one_shot / two_shot / nvls / local)."""
        from tridist_b200.ops.gemm_allreduce import pick_mode
        return pick_mode(self.ctx, self.M)

    def roof(self):
        from tridist_b200.ops.gemm_allreduce import pick_mode
        two = pick_mode(self.ctx, self.M) in ("two_shot", "nvls")
        return roofline.gemm_ar_roof(self.M, self.N, self.k_loc, self.R, two_shot=two)

    def check(self):
        self.run()
        rows = _sample_rows(self.M, 1, per_rank=min(32, self.M))
        ref = _sum_over_ranks(_matmul_fp32_rows(self.a[rows], self.b), self.R)
        return _rel_err(self.c[rows], ref)


class MoE(Workload):
    launches_per_run = 3

    def __init__(self, rank, R, zipf=0.0, E=64, H=4096, T=4096, topk=8, dtype=torch.float16):
        self.name = "moe_a2a_zipf" if zipf > 0 else "moe_a2a_uniform"
        self.R, self.T, self.H, self.topk = R, T, H, topk
        tokens, idx, wts = moe_inputs(rank, T, H, E, topk, 0, dtype, zipf)
        self.tok_host, self.idx_host, self.w_host = tokens.pin_memory(), idx.pin_memory(), wts.pin_memory()
        self.tokens, self.idx, self.wts = self.tok_host.cuda(), self.idx_host.cuda(), self.w_host.cuda()
        self.out = torch.empty_like(self.tokens)
        self.ctx = create_moe_a2a_intra_node_context(E, H, dtype, T, topk, rank, R)
        self.base = baselines.MoEBaseline(self.idx, E, H, R, dtype)
        self.h2d_bytes = tokens.numel() * 2 + idx.numel() * 4 + wts.numel() * 4
        # identity expert (as in the NCCL baseline, which sends the received rows straight back):
        # the expert-output buffer aliases the receive buffer, so no copy stands in for the expert
        self.ctx.out_buf, self.ctx.out = self.ctx.recv_buf, self.ctx.recv

    def run(self):
        moe_dispatch_intra_node_op(self.tokens, self.idx, self.ctx)
        moe_combine_intra_node_op(self.ctx, self.idx, self.out, self.wts)

    def baseline(self):
        return self.base()

    def stage(self):
        self.tokens.copy_(self.tok_host, non_blocking=True)
        self.idx.copy_(self.idx_host, non_blocking=True)
        self.wts.copy_(self.w_host, non_blocking=True)

    def digest(self):
        return self.out[0, :8].float().sum()

    def roof(self):
        # the busiest rank bounds the round: rows it receives (dispatch) and serves (combine)
        r = roofline.moe_roof(self.T, self.H, self.topk, self.R)
        if self.R > 1:
            hot = max(self.base.recv_splits_remote_rows, self.base.send_splits_remote_rows)
            r = roofline.roof_ms(0.0, 2.0 * hot * self.H * 2)
        return r

    def check(self):
        self.run()
        # identity expert and weights summing to one: combine returns the tokens
        return _rel_err(self.out, self.tokens.float())


class TPMLPLayer(Workload):
    launches_per_run = 2
    tol = 3e-2                  # bf16 results; the activation is rounded to bf16 between the two GEMMs

    def __init__(self, rank, R, M=8192, K=8192, I=28672, dtype=torch.bfloat16):
        self.name = "tp_mlp"
        self.rank = rank
        self.R, self.M, self.K, self.i_loc = R, M, K, I // R
        m_pr = M // R
        self.x_host = _pinned_randn((m_pr, K), 41 + rank, 1.0, dtype)
        self.x = self.x_host.cuda()
        self.w_gu = _dev_randn((2 * self.i_loc, K), 401 + rank, 0.02, dtype)
        self.w_down = _dev_randn((K, self.i_loc), 501 + rank, 0.02, dtype)
        cfg = TPMLPConfig(hidden=K, intermediate=I, max_tokens=M, dtype=dtype, mode="ag_rs", fuse_swiglu=True)
        self.layer = TPMLP(cfg, rank, R, self.w_gu, self.w_down)
        self.base = baselines.TPMLPBaseline(M, K, self.i_loc, R, dtype)
        self.y = None
        self.h2d_bytes = self.x_host.numel() * 2

    def run(self):
        self.y = self.layer(self.x)

    def baseline(self):
        return self.base(self.x, self.w_gu, self.w_down)

    def stage(self):
        self.x.copy_(self.x_host, non_blocking=True)

    def digest(self):
        return self.y[0, :8].float().sum()

    def roof(self):
        r1 = roofline.ag_gemm_roof(self.M, self.K, 2 * self.i_loc, self.R)
        r2 = roofline.gemm_rs_roof(self.M, self.K, self.i_loc, self.R)
        return {"ms": r1["ms"] + r2["ms"], "peaks": r1["peaks"]}

    def check(self):
        self.run()
        rows = _sample_rows(self.M, self.R)
        m_pr = self.M // self.R
        x_rows = torch.zeros((len(rows), self.K), dtype=torch.float32, device="cuda")
        for i, g in enumerate(rows):
            if g // m_pr == self.rank:
                x_rows[i] = self.x[g - self.rank * m_pr].float()
        _sum_over_ranks(x_rows, self.R)
        h = _matmul_fp32_rows(x_rows, self.w_gu)
        h2 = torch.nn.functional.silu(h[:, :self.i_loc]) * h[:, self.i_loc:]
        ref = _sum_over_ranks(_matmul_fp32_rows(h2, self.w_down), self.R)
        mine = [i for i, g in enumerate(rows) if g // m_pr == self.rank]
        return _rel_err(self.y[[rows[i] - self.rank * m_pr for i in mine]], ref[mine])


def build_all(rank: int, R: int, only: Optional[List[str]] = None) -> List[Workload]:
    makers: Dict[str, Callable[[], Workload]] = {
        "ag_gemm": lambda: AGGemm(rank, R),
        "gemm_rs": lambda: GemmRS(rank, R),
        "gemm_ar_m128": lambda: GemmAR(rank, R, 128),
        "gemm_ar_m1024": lambda: GemmAR(rank, R, 1024),
        "gemm_ar_m4096": lambda: GemmAR(rank, R, 4096),
        # 32768 tokens in total (4096 per rank at 8 GPUs, the named configuration): the step's
        # total work stays fixed as the GPU count changes
        "moe_a2a_uniform": lambda: MoE(rank, R, 0.0, T=32768 // R),
        "moe_a2a_zipf": lambda: MoE(rank, R, 1.2, T=32768 // R),
        "tp_mlp": lambda: TPMLPLayer(rank, R),
    }
    names = only or list(makers)
    return [makers[n]() for n in names]
