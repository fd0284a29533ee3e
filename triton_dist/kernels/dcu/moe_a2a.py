"""Alias of tridist_b200.ops.moe_a2a."""
from tridist_b200.ops.moe_a2a import *  # noqa: F401,F403
from tridist_b200.ops import moe_a2a as _m

globals().update({k: v for k, v in vars(_m).items() if not k.startswith("__")})
