"""tridist_b200 — Blackwell-native fused communication + compute operators.

Public API mirrors the reference library (create_*_context / *_op functions);
see the modules under ``tridist_b200.ops``.
"""
__version__ = "0.1.0"
