"""Alias of tridist_b200.parallel.predictor."""
from tridist_b200.parallel.predictor import StickyOrderPredictor, infer_straggler  # noqa: F401
