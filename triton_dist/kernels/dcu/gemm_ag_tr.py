"""Alias of tridist_b200.ops.gemm_ag_tr."""
from tridist_b200.ops.gemm_ag_tr import *  # noqa: F401,F403
from tridist_b200.ops import gemm_ag_tr as _m

globals().update({k: v for k, v in vars(_m).items() if not k.startswith("__")})
