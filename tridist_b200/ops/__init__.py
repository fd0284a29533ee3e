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
from .ag_tr_pred import (I1PredContext, calibrate_sleep_cycles_per_us, create_i1_context,  # noqa: F401
                         finalize_i1_context, i1_ag_tr, i1_ag_tr_op, i1_observer_read, i1_table_peek,
                         i1_table_write, observed_straggler)
from .gemm_ag_tr import (create_gemm_ag_tr_context, finalize_gemm_ag_tr_context, gemm_ag_tr,  # noqa: F401
                         gemm_ag_tr_op)
from .gemm_ar_pred import gemm_ar_pred_op, make_gate_flag, task_events  # noqa: F401
from .gemm_ar_rd import (create_gemm_ar_rd_context, finalize_gemm_ar_rd_context, gemm_ar_rd,  # noqa: F401
                         gemm_ar_rd_op)
from .gemm_rs_v5 import (create_gemm_rs_v5_context, finalize_gemm_rs_v5_context, gemm_rs_v5,  # noqa: F401
                         gemm_rs_v5_op)
# the arrival-order predictor of the skew layer (reference: triton_dist/kernels/dcu/i1_predictor.py:35)
from ..parallel.predictor import StickyOrderPredictor, infer_straggler  # noqa: F401,E402
