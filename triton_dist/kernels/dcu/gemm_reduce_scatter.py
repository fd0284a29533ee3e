"""Alias of tridist_b200.ops.gemm_reduce_scatter."""
from tridist_b200.ops.gemm_reduce_scatter import *  # noqa: F401,F403
from tridist_b200.ops import gemm_reduce_scatter as _m

globals().update({k: v for k, v in vars(_m).items() if not k.startswith("__")})
