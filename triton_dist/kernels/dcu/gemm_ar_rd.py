"""Alias of tridist_b200.ops.gemm_ar_rd."""
from tridist_b200.ops.gemm_ar_rd import *  # noqa: F401,F403
from tridist_b200.ops import gemm_ar_rd as _m

globals().update({k: v for k, v in vars(_m).items() if not k.startswith("__")})
