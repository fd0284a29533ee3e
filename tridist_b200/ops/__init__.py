"""Operator API (same names and signatures as the reference's triton_dist.kernels.dcu)."""
from .all_gather_gemm import (AllGatherGEMMTensorParallelContext, ag_gemm_intra_node,  # noqa: F401
                              ag_gemm_intra_node_op, create_ag_gemm_intra_node_context,
                              finalize_ag_gemm_context)
from .gemm_allreduce import (GemmARContext, create_gemm_ar_intra_node_context,  # noqa: F401
                             finalize_gemm_ar_context, gemm_ar_intra_node, gemm_ar_intra_node_op)
from .gemm_reduce_scatter import (GemmRSContext, create_gemm_rs_intra_node_context,  # noqa: F401
                                  finalize_gemm_rs_context, gemm_rs_intra_node, gemm_rs_intra_node_op)
from .moe_a2a import (MoEA2AContext, create_moe_a2a_intra_node_context,  # noqa: F401
                      finalize_moe_a2a_context, moe_combine_intra_node_op, moe_dispatch_intra_node_op)
from .swiglu import swiglu  # noqa: F401
