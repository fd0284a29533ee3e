"""Tensor-parallel SwiGLU MLP layer built from the fused operators.

The reference composes this layer only in a benchmark script
(bench/s21_bench_tp_mlp_dcu.py:156-364); here it is a reusable module with the
same two modes and the same weight layouts:

ag_rs    x_loc [M/R, K]  --AG+GEMM-->  h [M, 2I/R]  (gate_up shard = [I/R gate | I/R up])
         --SwiGLU-->  h2 [M, I/R]  --GEMM+RS (W_down shard [K, I/R])-->  y_loc [M/R, K]
gemm_ar  x_k [M, K/R]  --GEMM+AR (W_gu [2I, K/R])-->  h [M, 2I] on every rank (global layout:
         rank-blocked [I/R gate | I/R up] per shard)  --SwiGLU + own slice-->  a2 [M, I/R]
         --GEMM+AR (W_down [K, I/R])-->  y [M, K] on every rank

With ``fuse_swiglu=True`` (ag_rs mode) the activation runs in the AG+GEMM
epilogue and h is never written to memory.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from ..ops import (ag_gemm_intra_node_op, create_ag_gemm_intra_node_context,
                   create_gemm_ar_intra_node_context, create_gemm_rs_intra_node_context,
                   gemm_ar_intra_node_op, gemm_rs_intra_node_op, swiglu)

LAYER_CONFIGS: Dict[str, Dict[str, int]] = {
    "LLaMA-7B": dict(I=11008, K=4096),
    "LLaMA-3.1-70B": dict(I=28672, K=8192),
    "LLaMA-3.1-405B": dict(I=53248, K=16384),
    "Qwen2-72B": dict(I=29568, K=8192),
    "GPT-3-175B": dict(I=49152, K=12288),
}


@dataclass
class TPMLPConfig:
    hidden: int                 # K
    intermediate: int           # I
    max_tokens: int             # M (global)
    dtype: torch.dtype = torch.bfloat16
    mode: str = "ag_rs"         # "ag_rs" | "gemm_ar"
    fuse_swiglu: bool = True


class TPMLP:
    """One rank's shard of the layer. ``w_gate_up`` is [2I/R, K] (ag_rs) or [2I, K/R]
    (gemm_ar); ``w_down`` is [K, I/R] in both modes."""

    def __init__(self, cfg: TPMLPConfig, rank: int, num_ranks: int, w_gate_up: torch.Tensor,
                 w_down: torch.Tensor, world=None):
        self.cfg, self.rank, self.R = cfg, rank, num_ranks
        self.w_gate_up, self.w_down = w_gate_up, w_down
        K, I, M = cfg.hidden, cfg.intermediate, cfg.max_tokens
        assert I % num_ranks == 0 and M % num_ranks == 0
        self.i_loc = I // num_ranks
        dev = w_gate_up.device
        if cfg.mode == "ag_rs":
            assert tuple(w_gate_up.shape) == (2 * self.i_loc, K) and tuple(w_down.shape) == (K, self.i_loc)
            m_pr = M // num_ranks
            chunk = m_pr if m_pr % 128 == 0 else 128
            self.ag = create_ag_gemm_intra_node_context(M, K, cfg.dtype, cfg.dtype, rank, num_ranks,
                                                        M_PER_CHUNK=chunk, world=world)
            self.rs = create_gemm_rs_intra_node_context(M, K, cfg.dtype, rank, num_ranks, world=world)
            self.h = None if cfg.fuse_swiglu else torch.empty((M, 2 * self.i_loc), dtype=cfg.dtype, device=dev)
            self.h2 = torch.empty((M, self.i_loc), dtype=cfg.dtype, device=dev)
            self.y = torch.empty((m_pr, K), dtype=cfg.dtype, device=dev)
        elif cfg.mode == "gemm_ar":
            assert tuple(w_gate_up.shape) == (2 * I, K // num_ranks) and tuple(w_down.shape) == (K, self.i_loc)
            self.ar1 = create_gemm_ar_intra_node_context(M, 2 * I, cfg.dtype, cfg.dtype, rank, num_ranks,
                                                         M_PER_CHUNK=64, world=world)
            self.ar2 = create_gemm_ar_intra_node_context(M, K, cfg.dtype, cfg.dtype, rank, num_ranks,
                                                         M_PER_CHUNK=64, world=world)
            self.h = torch.empty((M, 2 * I), dtype=cfg.dtype, device=dev)
            self.h2 = torch.empty((M, self.i_loc), dtype=cfg.dtype, device=dev)
            self.y = torch.empty((M, K), dtype=cfg.dtype, device=dev)
        else:
            raise ValueError(f"unknown mode {cfg.mode!r}")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if cfg.mode == "ag_rs":
            m_pr = x.shape[0]
            M = m_pr * self.R
            h2 = self.h2[:M]
            if cfg.fuse_swiglu and x.is_cuda:
                ag_gemm_intra_node_op(x, self.w_gate_up, h2, self.ag, fuse_swiglu=True)
            else:
                if self.h is None:
                    self.h = torch.empty((cfg.max_tokens, 2 * self.i_loc), dtype=cfg.dtype, device=x.device)
                h = self.h[:M]
                ag_gemm_intra_node_op(x, self.w_gate_up, h, self.ag)
                swiglu(h, h2)
            return gemm_rs_intra_node_op(h2, self.w_down, cfg.dtype, self.rank, self.R, self.rs,
                                         out=self.y[:m_pr]) if x.is_cuda else \
                gemm_rs_intra_node_op(h2, self.w_down, cfg.dtype, self.rank, self.R, self.rs)
        M = x.shape[0]
        h = self.h[:M]
        gemm_ar_intra_node_op(x, self.w_gate_up, h, self.ar1)
        # own rank-blocked [gate | up] block of the global layout
        blk = h[:, self.rank * 2 * self.i_loc:(self.rank + 1) * 2 * self.i_loc]
        h2 = swiglu(blk, self.h2[:M])
        y = self.y[:M]
        gemm_ar_intra_node_op(h2, self.w_down, y, self.ar2)
        return y

    __call__ = forward

    def close(self) -> None:
        """Collective: release the symmetric buffers of the layer's operator contexts."""
        from ..ops import finalize_ag_gemm_context, finalize_gemm_ar_context, finalize_gemm_rs_context
        if self.cfg.mode == "ag_rs":
            finalize_ag_gemm_context(self.ag)
            finalize_gemm_rs_context(self.rs)
        else:
            finalize_gemm_ar_context(self.ar1)
            finalize_gemm_ar_context(self.ar2)


def reference_forward(x_full: torch.Tensor, w_gu_shards, w_down_shards) -> torch.Tensor:
    """fp32 reference of the ag_rs layout: shards are per-rank [2I/R, K] and [K, I/R]."""
    R = len(w_gu_shards)
    xf = x_full.float()
    y = None
    for r in range(R):
        h = xf @ w_gu_shards[r].float().t()
        i_loc = h.shape[1] // 2
        h2 = torch.nn.functional.silu(h[:, :i_loc]) * h[:, i_loc:]
        part = h2 @ w_down_shards[r].float().t()
        y = part if y is None else y + part
    return y
