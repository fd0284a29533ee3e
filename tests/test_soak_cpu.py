"""The numerical soak (bench/soak_ops.py) on the gloo oracle backend: several rounds on one
context per operator with fresh data, world size 2."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _soak(rank, R):
    from bench.soak_ops import soak
    from tridist_b200.parallel.runtime import CpuWorld
    worst, problems = soak(rank, R, CpuWorld(rank, R), rounds=4, small=True, dtype=torch.float32, tol=1e-4)
    assert not problems, problems
    assert set(worst) == {"ag", "rs", "ar", "moe"}


def test_soak_two_cpu_ranks():
    from tridist_b200.utils.testing import spawn
    spawn(_soak, 2, backend="gloo", timeout=240)


def test_soak_reports_bad_rows():
    from bench.soak_ops import _report
    problems = []
    ref = torch.zeros(8, 4)
    got = ref.clone()
    got[5, 2] = 1.0
    assert _report(problems, "x", 7, got, ref, 1e-2) == 1.0
    assert problems == [{"op": "x", "round": 7, "max_abs_err": 1.0, "bad_rows": [5], "n_bad_rows": 1}]
    assert _report(problems, "x", 8, ref, ref, 1e-2) == 0.0 and len(problems) == 1
