"""Alias of tridist_b200.ops.gemm_rs_v5."""
from tridist_b200.ops.gemm_rs_v5 import *  # noqa: F401,F403
from tridist_b200.ops import gemm_rs_v5 as _m

globals().update({k: v for k, v in vars(_m).items() if not k.startswith("__")})
