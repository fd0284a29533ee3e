"""Alias of tridist_b200.ops.ag_tr_pred."""
from tridist_b200.ops.ag_tr_pred import *  # noqa: F401,F403
from tridist_b200.ops import ag_tr_pred as _m

globals().update({k: v for k, v in vars(_m).items() if not k.startswith("__")})
