"""Model-level building blocks made of the fused operators."""
from .tp_mlp import LAYER_CONFIGS, TPMLP, TPMLPConfig, reference_forward  # noqa: F401
