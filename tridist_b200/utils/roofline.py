"""Roofline arithmetic for the fused operators.

The target time of a fused compute+collective kernel is the slower of
(FLOPs / measured GEMM peak) and (bytes that must cross NVLink / link bandwidth
per direction per GPU); the reported fraction is target / measured.  Peaks come
from ``MEASURED_PEAKS.json`` at the repository root when present.
"""
from __future__ import annotations

import json
import os
from typing import Dict

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NVLINK_GBS_PER_DIR = 770.0      # measured peer copy, per direction per GPU (900 nominal)


def load_peaks() -> Dict:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        d["source"] = "measured"
        return d
    d = dict(FALLBACK)
    d["source"] = "fallback"
    return d


def roof_ms(flops: float, nvlink_bytes: float, hbm_bytes: float = 0.0, sustained: bool = False) -> Dict:
    p = load_peaks()
    tf = p["bf16_tflops_sustained"] if sustained else p["bf16_tflops"]
    t_flops = flops / (tf * 1e12) * 1e3
    t_link = nvlink_bytes / (NVLINK_GBS_PER_DIR * 1e9) * 1e3
    t_hbm = hbm_bytes / (p["hbm_gbs"] * 1e9) * 1e3
    return {"ms": max(t_flops, t_link, t_hbm), "flops_ms": t_flops, "nvlink_ms": t_link, "hbm_ms": t_hbm,
            "peaks": p["source"]}


def ag_gemm_roof(M, K, n_loc, R):
    return roof_ms(2.0 * M * K * n_loc, (R - 1) * (M // R) * K * 2)


def gemm_rs_roof(M, N, k_loc, R):
    return roof_ms(2.0 * M * N * k_loc, (R - 1) * (M // R) * N * 2)


def gemm_ar_roof(M, N, k_loc, R, two_shot=True):
    part = M * N * 2
    link = 2 * (R - 1) * part / R if two_shot else (R - 1) * part
    return roof_ms(2.0 * M * N * k_loc, link)


def moe_roof(T, H, topk, R):
    one_way = T * topk * H * 2 * (R - 1) / max(R, 1)
    # dispatch then combine: each direction carries the rows once; at R = 1 it is an HBM copy
    return roof_ms(0.0, 2 * one_way if R > 1 else 0.0, hbm_bytes=4.0 * T * topk * H * 2)
