"""Same re-exports as the reference package (triton_dist/kernels/dcu/__init__.py:26-44)."""
from tridist_b200.ops import (ag_gemm_intra_node, ag_gemm_intra_node_op, create_ag_gemm_intra_node_context,  # noqa: F401
                              create_gemm_rs_intra_node_context, gemm_rs_intra_node, gemm_rs_intra_node_op)

__all__ = ["ag_gemm_intra_node", "ag_gemm_intra_node_op", "create_ag_gemm_intra_node_context",
           "gemm_rs_intra_node", "gemm_rs_intra_node_op", "create_gemm_rs_intra_node_context"]
