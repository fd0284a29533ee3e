"""Secondary entry points (tile-ready AG, windowed RS, recursive-doubling AR, I1 layer,
order-driven AR carrier, TP-MLP layer) on the CPU/gloo backend at world size 2, with the
round pattern of the reference's tests (tests/test_gemm_rs_v5.py:89-105): a few full
rounds with fresh data, then the GEMM-only decomposition."""
import torch

from tridist_b200.utils.testing import ks_inputs, randn_seeded, spawn


def _rounds(rank, R):
    from tridist_b200.ops import (create_gemm_ag_tr_context, create_gemm_ar_rd_context, create_gemm_rs_v5_context,
                                  create_i1_context, finalize_gemm_ag_tr_context, finalize_gemm_ar_rd_context,
                                  finalize_gemm_rs_v5_context, finalize_i1_context, gemm_ag_tr, gemm_ag_tr_op,
                                  gemm_ar_pred_op, gemm_ar_rd, gemm_ar_rd_op, gemm_rs_v5, gemm_rs_v5_op, i1_ag_tr,
                                  i1_observer_read, i1_table_peek, i1_table_write)
    from tridist_b200.parallel.predictor import StickyOrderPredictor
    from tridist_b200.parallel.runtime import CpuWorld
    w = CpuWorld(rank, R)
    f32 = torch.float32
    m_pr, K, N = 128, 64, 128
    ag = create_gemm_ag_tr_context(m_pr * R, K, f32, f32, rank, R, world=w)
    ic = create_i1_context(m_pr * R, K, f32, f32, rank, R, world=w)
    pred = StickyOrderPredictor(rank, R)
    for it in range(3):
        a_all = [randn_seeded((m_pr, K), 10 * it + s, 0.1) for s in range(R)]
        b = randn_seeded((N, K), 500 + it + rank, 0.1)
        ref = torch.cat(a_all, 0) @ b.t()
        c = gemm_ag_tr(a_all[rank], b, ag)
        assert (c - ref).abs().max().item() < 1e-4
        c2 = torch.empty_like(c)
        gemm_ag_tr_op(a_all[rank], b, c2, ag, component="gemm")
        assert torch.equal(c, c2)
        pred.observe((rank + 1) % R)
        t = pred.table(k_eff=1)
        i1_table_write(ic, t["seq"], t["degraded"], t["mode"], t["order_packed"], t["k_eff"])
        words = i1_table_peek(ic)
        assert words[0] == t["seq"] and words[2] == t["mode"] and words[4:4 + R] == t["order"]
        c3 = i1_ag_tr(a_all[rank], b, ic)
        assert (c3 - ref).abs().max().item() < 1e-4
        obs = i1_observer_read(ic)
        assert len(obs) == 1 + 2 * R and obs[1] == rank
    M, kl = 128, 48
    rs = create_gemm_rs_v5_context(M, N, f32, rank, R, world=w)
    ar = create_gemm_ar_rd_context(M, 128, f32, f32, rank, R, world=w)
    for it in range(3):
        a_all, b_all = ks_inputs(R, M, N, kl, it, f32, 0.1)
        ref = sum(a_all[s] @ b_all[s].t() for s in range(R))
        out = gemm_rs_v5(a_all[rank], b_all[rank], rs)
        mp = M // R
        assert (out - ref[rank * mp:(rank + 1) * mp]).abs().max().item() < 1e-4
        g = torch.empty_like(out)
        gemm_rs_v5_op(a_all[rank], b_all[rank], g, rs, component="gemm")
        assert (g - (a_all[rank] @ b_all[rank].t())[rank * mp:(rank + 1) * mp]).abs().max().item() < 1e-4
        a2, b2 = ks_inputs(R, M, 128, kl, 50 + it, f32, 0.1)
        ref2 = sum(a2[s] @ b2[s].t() for s in range(R))
        c = gemm_ar_rd(a2[rank], b2[rank], ar)
        assert (c - ref2).abs().max().item() < 1e-4
        cg = torch.empty_like(c)
        gemm_ar_rd_op(a2[rank], b2[rank], cg, ar, component="gemm")
        assert (cg - a2[rank] @ b2[rank].t()).abs().max().item() < 1e-4
        # order-driven carrier: panels of 64 rows in reversed order give the same result
        ar.chunk_rows = 64
        cp = torch.empty_like(c)
        gemm_ar_pred_op(a2[rank], b2[rank], cp, ar, order=[1, 0])
        assert (cp - ref2).abs().max().item() < 1e-4
    for fin, ctx in ((finalize_gemm_ag_tr_context, ag), (finalize_i1_context, ic),
                     (finalize_gemm_rs_v5_context, rs), (finalize_gemm_ar_rd_context, ar)):
        fin(ctx)


def _tp_mlp(rank, R):
    from tridist_b200.models.tp_mlp import TPMLP, TPMLPConfig, reference_forward
    from tridist_b200.parallel.runtime import CpuWorld
    w = CpuWorld(rank, R)
    M, K, I = 256, 128, 64
    i_loc = I // R
    x_all = [randn_seeded((M // R, K), 70 + s, 1.0) for s in range(R)]
    wgu = [randn_seeded((2 * i_loc, K), 80 + s, 0.2) for s in range(R)]
    wd = [randn_seeded((K, i_loc), 90 + s, 0.2) for s in range(R)]
    ref = reference_forward(torch.cat(x_all, 0), wgu, wd)
    layer = TPMLP(TPMLPConfig(hidden=K, intermediate=I, max_tokens=M, dtype=torch.float32, mode="ag_rs"),
                  rank, R, wgu[rank], wd[rank], world=w)
    y = layer(x_all[rank])
    mp = M // R
    assert (y - ref[rank * mp:(rank + 1) * mp]).abs().max().item() < 1e-4
    # gemm_ar mode: K-sharded input, global rank-blocked [gate | up] layout of W_gu
    xk = torch.cat(x_all, 0)[:, rank * (K // R):(rank + 1) * (K // R)].contiguous()
    wgu_full = torch.cat(wgu, 0)                      # [2I, K], rank-blocked
    wgu_k = wgu_full[:, rank * (K // R):(rank + 1) * (K // R)].contiguous()
    layer2 = TPMLP(TPMLPConfig(hidden=K, intermediate=I, max_tokens=M, dtype=torch.float32, mode="gemm_ar"),
                   rank, R, wgu_k, wd[rank], world=w)
    y2 = layer2(xk)
    assert (y2 - ref).abs().max().item() < 1e-4


def test_secondary_api_ws2():
    spawn(_rounds, 2)


def test_secondary_api_ws1():
    _rounds(0, 1)


def test_tp_mlp_ws2():
    spawn(_tp_mlp, 2)
