"""SwiGLU: ``out = silu(h[:, :I]) * h[:, I:]`` for gate/up halves stored side by side.

The reference has no kernel for this; its TP-MLP bench calls ``F.silu(gate) * up``
between the two fused GEMMs, with gate/up laid out rank-blocked per shard
(bench/s21_bench_tp_mlp_dcu.py:21-22, 206-207). Here it is one memory-bound
sm_100a kernel, and it can also be folded into the AG+GEMM epilogue
(``ag_gemm_intra_node_op(..., fuse_swiglu=True)``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from ..parallel.runtime import native
from ._gemm_common import is_bf16


def swiglu(h: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    assert h.dim() == 2 and h.shape[1] % 2 == 0 and h.stride(1) == 1
    rows, two_i = h.shape
    inter = two_i // 2
    if not h.is_cuda:
        res = (F.silu(h[:, :inter].float()) * h[:, inter:].float()).to(h.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is None:
        out = torch.empty((rows, inter), dtype=h.dtype, device=h.device)
    assert out.is_contiguous()
    native().swiglu(h.data_ptr(), out.data_ptr(), rows, inter, h.stride(0), is_bf16(h.dtype))
    return out
