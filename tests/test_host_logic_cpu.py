"""Host-side decisions that need no GPU: all-reduce algorithm choice, clock-sample windows,
worlds without a multicast mapping, and the reference's import paths."""
import types

import torch


def _ar_ctx(R, mode="auto", mc=None, max_M=4096, N=8192):
    from tridist_b200.ops.gemm_allreduce import GemmARContext
    return GemmARContext(rank=0, num_ranks=R, max_M=max_M, N=N, input_dtype=torch.float16,
                         output_dtype=torch.float16, M_PER_CHUNK=64, world=None, mode=mode, mc=mc)


def test_allreduce_mode_choice(monkeypatch):
    from tridist_b200.ops.gemm_allreduce import pick_mode
    for name in ("TRIDIST_AR_NVLS_MIN_BYTES", "TRIDIST_AR_ONE_SHOT_BYTES"):
        monkeypatch.delenv(name, raising=False)
    assert pick_mode(_ar_ctx(1), 128) == "local"
    assert pick_mode(_ar_ctx(2), 4096) == "one_shot"                  # same bytes, one hop less
    assert pick_mode(_ar_ctx(8), 128) == "one_shot"                   # 2 MiB partial, no multicast buffer
    assert pick_mode(_ar_ctx(8), 4096) == "two_shot"
    mc = types.SimpleNamespace(mc_ptr=1 << 40)
    assert pick_mode(_ar_ctx(8, mc=mc), 128) == "nvls"
    assert pick_mode(_ar_ctx(2, mc=mc), 4096) == "one_shot"           # two ranks never go through the switch
    assert pick_mode(_ar_ctx(8, mode="two_shot", mc=mc), 4096) == "two_shot"   # explicit mode wins
    import pytest
    with pytest.raises(RuntimeError):
        pick_mode(_ar_ctx(8, mode="nvls"), 128)                      # asked for, but no multicast buffer
    monkeypatch.setenv("TRIDIST_AR_NVLS_MIN_BYTES", str(8 << 20))
    assert pick_mode(_ar_ctx(8, mc=mc), 128) == "one_shot"            # below the switch threshold
    assert pick_mode(_ar_ctx(8, mc=mc), 4096) == "nvls"


def test_clock_sampler_window():
    from tridist_b200.utils.timing import ClockSampler
    s = ClockSampler(0)
    row = "0, {}, 1965, 900.0, 0x4, Not Active, Not Active, Not Active, {}"
    s.lines = [row.format(600, "Not Active"), row.format(1400, "Active"), row.format(1500, "Active"),
               row.format(700, "Not Active")]
    s.stamps = [1.0, 2.0, 2.5, 4.0]
    inside = s.stop(window=(1.9, 2.6))
    assert inside["samples"] == 2 and inside["sm_mhz"] == 1450.0 and inside["reasons"] == ["sw_power_cap"]
    assert inside["window"] == "timed region"
    short = s.stop(window=(2.1, 2.2))            # nothing arrived inside: fall back to everything since start()
    assert short["samples"] == 4 and "warm-up" in short["window"]
    assert s.stop()["samples"] == 4


def test_worlds_without_multicast():
    from tridist_b200.parallel.runtime import CpuWorld
    w = CpuWorld(0, 1)
    assert w.alloc_multicast(1 << 20) is None
    w.release_multicast()                        # no-op, must not raise


def test_reference_import_paths():
    import pydushmem
    import triton_dist.kernels.dcu as dcu
    from triton_dist.kernels.dcu import gemm_allreduce, i1_predictor, moe_a2a
    import tridist_b200.ops as ops
    assert dcu.ag_gemm_intra_node_op is ops.ag_gemm_intra_node_op
    assert gemm_allreduce.gemm_ar_intra_node is ops.gemm_ar_intra_node
    assert moe_a2a.moe_dispatch_intra_node_op is ops.moe_dispatch_intra_node_op
    assert i1_predictor.StickyOrderPredictor is ops.StickyOrderPredictor
    from triton_dist.kernels.dcu import common_ops
    for name in ("init_dcu", "dcu_state", "memcpy_async", "fan_out_memcpy_async", "set_signal", "wait_eq",
                 "SymmBarrier", "barrier_all_on_stream"):
        assert callable(getattr(common_ops, name)), name
    assert pydushmem.host.mpi_comm_size() >= 1
    assert pydushmem.get_uniqueid()
    for name in ("malloc", "calloc", "align", "free", "ptr", "putmem", "putmem_nbi", "getmem", "getmem_nbi", "quiet",
                 "fence", "barrier_all", "my_pe", "n_pes", "finalize"):
        assert callable(getattr(pydushmem, name))
        from tridist_b200.parallel.symm_host import SymmHost
        assert hasattr(SymmHost, name), name          # the delegate names a real method


def test_ticket_ceiling_and_ignored_argument_warnings():
    import warnings

    import pytest
    import torch

    from tridist_b200.ops import create_gemm_ar_rd_context, create_gemm_rs_v5_context
    from tridist_b200.ops._gemm_common import MAX_TICKETS, next_round
    from tridist_b200.parallel.runtime import CpuWorld
    assert next_round(41) == 42
    with pytest.raises(RuntimeError, match="create a new one"):
        next_round(MAX_TICKETS - 1, "reduce-scatter context")
    w = CpuWorld(0, 1)
    with pytest.warns(UserWarning, match="wait_mode='spin' has no effect"):
        create_gemm_ar_rd_context(256, 128, torch.float32, torch.float32, 0, 1, wait_mode="spin", world=w)
    with warnings.catch_warnings():
        warnings.simplefilter("error")                 # defaults and honoured arguments stay silent
        ctx = create_gemm_ar_rd_context(256, 128, torch.float32, torch.float32, 0, 1, chunk_rows=64, stage_slots=3,
                                        world=w)
        assert ctx.chunk_rows == 64 and ctx.rd.stage_slots == 3 and ctx.rd.num_chunks == 4
        rs = create_gemm_rs_v5_context(256, 128, torch.float32, 0, 1, steady_sms=16, tail_chunk_window=2,
                                       chunk_rows=128, world=w)
        assert rs.reduce_ctas == 16 and rs.reduce_tail == 2
    with pytest.warns(UserWarning, match="comm_lanes=4"):
        create_gemm_rs_v5_context(256, 128, torch.float32, 0, 1, comm_lanes=4, world=w)


def test_recursive_doubling_panels_partners_and_tickets():
    """Host arithmetic of the panel exchange (reference rules: gemm_ar_rd.py:317-329 panel rows,
    :424-426 XOR partners, ticket = round_base + task + 1 with a per-call stride)."""
    import torch

    from tridist_b200.ops.gemm_ar_rd import (MAX_TICKETS, _advance, create_gemm_ar_rd_context, panel_rows,
                                             partners_of)
    from tridist_b200.parallel.runtime import CpuWorld
    assert partners_of(5, 8) == [4, 7, 1] and partners_of(1, 2) == [0] and partners_of(0, 1) == []
    assert panel_rows(4096, 8192) == 512                      # 8 MB cap: 8 MB / (8192 * 2 B) = 512 rows
    assert panel_rows(4096, 1024) == 1024                     # four panels
    assert panel_rows(1024, 1024) == 512                      # not below min_chunk_rows
    assert panel_rows(256, 1024) == 256                       # never above max_M
    assert panel_rows(4096, 1024, chunk_rows=200) == 192      # caller's value, 64-row aligned
    ctx = create_gemm_ar_rd_context(1024, 256, torch.float32, torch.float32, 0, 1, chunk_rows=256, stage_slots=2,
                                    world=CpuWorld(0, 1))
    rd = ctx.rd
    assert (rd.num_chunks, rd.stage_slots, rd.round_stride, rd.phases) == (4, 2, 5, 0)
    assert _advance(ctx, 4) == 5 and _advance(ctx, 2) == 10   # the stride does not depend on the call's M
    rd.round_base = MAX_TICKETS - 6
    import pytest
    with pytest.raises(RuntimeError, match="ran out of tickets"):
        _advance(ctx, 4)


def test_plan_cache_is_lru_and_reports_thrashing(monkeypatch):
    """Plans are keyed by operand addresses: stable buffers hit, fresh addresses every call evict and
    (after a while) warn."""
    import warnings

    import pytest

    from tridist_b200.ops import _gemm_common as gc

    destroyed = []

    class FakeNative:
        @staticmethod
        def gemm_plan_destroy(pid):
            destroyed.append(pid)

    monkeypatch.setattr(gc, "native", lambda: FakeNative)
    made = []

    def maker(k):
        def make():
            made.append(k)
            return 100 + len(made)
        return make

    c = gc.PlanCache(capacity=2)
    a = c.get(("a",), maker("a"))
    b = c.get(("b",), maker("b"))
    assert c.get(("a",), maker("a")) == a and made == ["a", "b"] and (c.hits, c.misses) == (1, 2)
    c.get(("c",), maker("c"))                      # evicts b, the least recently used
    assert destroyed == [b] and c.evictions == 1
    assert c.get(("a",), maker("a")) == a          # still cached
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        for i in range(6):                         # 1 + 6 evictions < 4 * capacity: silent
            c.get(("x", i), maker(i))
    with pytest.warns(UserWarning, match="reuse buffers"):
        c.get(("x", 99), maker(99))
    c.clear()
    assert len(destroyed) == 1 + 7 + 2


def test_transfer_plans_of_the_all_gather():
    """How many CTAs carry the all-gather and how many rounds they sit out: the multicast form
    sends the shard once, so it needs fewer CTA-rounds than the bulk-copy push from three ranks on."""
    from tridist_b200.ops.all_gather_gemm import _push_plan
    M, K = 8192, 12288
    for R in (4, 8):
        n_pr, m_pr = 49152 // R, M // R
        mc = _push_plan(M, n_pr, K, m_pr, R, 256, multicast=True)
        push = _push_plan(M, n_pr, K, m_pr, R, 256)
        assert 4 <= mc[0] <= 16 and 4 <= push[0] <= 32 and mc[0] % 2 == 0 and push[0] % 2 == 0
        assert mc[0] * mc[1] <= push[0] * push[1], (R, mc, push)
    # a forced CTA count is honoured, the rounds follow from it
    assert _push_plan(M, 6144, K, 1024, 8, 256, want_ctas=12)[0] == 12


def test_report_tables_and_overrides(tmp_path):
    """bench/report.py: one recorded line per GPU count becomes the scaling table; an override file
    replaces the cells it holds, marks them and re-derives the geometric mean."""
    import json

    from bench.report import load, tables

    def line(n, ops, step):
        return {"n_gpus": n, "ms_per_step": step, "vs_baseline": 1.0, "e2e": {"value": 2 * step},
                "clocks": {"sm_mhz": 1500.0, "reasons": []},
                "ops": {k: {"fused_p50_ms": f, "cublas_nccl_p50_ms": b, "speedup_vs_cublas_nccl": round(b / f, 3),
                            "roofline_frac": 0.5} for k, (f, b) in ops.items()}}

    f1, f8, fo = tmp_path / "b1.json", tmp_path / "b8.json", tmp_path / "o8.json"
    f1.write_text(json.dumps(line(1, {"ag_gemm": (8.0, 8.0), "gemm_rs": (8.0, 8.8)}, 16.0)))
    f8.write_text(json.dumps(line(8, {"ag_gemm": (1.2, 1.14), "gemm_rs": (1.0, 1.1)}, 2.2)))
    fo.write_text(json.dumps(line(8, {"ag_gemm": (1.0, 1.14)}, 1.0)))
    runs = load([str(f8), str(f1)], [str(fo)])
    assert list(runs) == [1, 8]
    assert runs[8]["ops"]["ag_gemm"]["fused_p50_ms"] == 1.0 and runs[8]["ops"]["ag_gemm"]["overridden"]
    assert abs(runs[8]["vs_baseline"] - (1.14 * 1.1) ** 0.5) < 2e-3
    text = tables(runs)
    assert "| ag_gemm | 8.000 / 8.000 (1.00) | 1.000 / 1.140 (1.14) † | 0.5 |" in text
    assert "| 8 | 2.200 | 4.4 | 0.91 |" in text          # 16 / (2.2 * 8)
