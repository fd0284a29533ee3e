"""Alias of tridist_b200.ops.all_gather_gemm."""
from tridist_b200.ops.all_gather_gemm import *  # noqa: F401,F403
from tridist_b200.ops import all_gather_gemm as _m

globals().update({k: v for k, v in vars(_m).items() if not k.startswith("__")})
