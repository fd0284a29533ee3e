"""Single-GPU tests of the sm_100a kernels.

Numerics are compared against a plain fp32 PyTorch reference of the same op.
The cross-rank protocols (tickets, peer slots, segment tables) are exercised on
one GPU by running R virtual ranks inside one cooperative launch
(``EmulatedWorld``); real multi-process runs live in test_gpu_multi.py.
"""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _world1():
    from tridist_b200.parallel.runtime import ProcessWorld
    global _W1
    try:
        return _W1
    except NameError:
        _W1 = ProcessWorld(0, 1)
        return _W1


def _loaded_native():
    from tridist_b200.parallel.runtime import native
    C = native()
    assert C.__file__.endswith("_C.so")
    return C


TOL = 1e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape,bn", [((128, 256, 64), 256), ((256, 128, 192), 128), ((384, 640, 1000), None),
                                      ((1024, 2048, 512), None), ((192, 384, 520), 256)])
def test_plain_gemm(shape, bn, dtype):
    from tridist_b200.ops._gemm_common import gemm_nt
    _loaded_native()
    M, N, K = shape
    torch.manual_seed(1)
    a = (torch.randn(M, K, device="cuda") * 0.05).to(dtype)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(dtype)
    before = _loaded_native().launch_count()
    out = gemm_nt(a, b, bn=bn)
    torch.cuda.synchronize()
    assert _loaded_native().launch_count() == before + 1
    ref = a.float() @ b.float().t()
    assert (out.float() - ref).abs().max().item() < TOL


def test_gemm_swiglu_epilogue_and_kernel():
    from tridist_b200.ops import swiglu
    from tridist_b200.ops._gemm_common import gemm_nt
    torch.manual_seed(2)
    M, I, K = 512, 640, 384
    a = (torch.randn(M, K, device="cuda") * 0.1).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device="cuda") * 0.1).to(torch.bfloat16)
    h = a.float() @ w.float().t()
    ref = F.silu(h[:, :I]) * h[:, I:]
    fused = gemm_nt(a, w, swiglu=True)
    two_step = swiglu(gemm_nt(a, w))
    torch.cuda.synchronize()
    assert (fused.float() - ref).abs().max().item() < TOL
    assert (two_step.float() - ref).abs().max().item() < 3e-2   # h rounded to bf16 first
    # stand-alone kernel against torch on the same 16-bit input
    hh = (torch.randn(300, 2 * 264, device="cuda")).to(torch.float16)
    got = swiglu(hh)
    exp = (F.silu(hh[:, :264].float()) * hh[:, 264:].float())
    assert (got.float() - exp).abs().max().item() < 1e-2


def test_public_api_single_rank():
    """R = 1 degenerates: every op collapses to the local GEMM / permutation."""
    from tridist_b200.ops import (ag_gemm_intra_node, create_ag_gemm_intra_node_context,
                                  create_gemm_ar_intra_node_context, create_gemm_rs_intra_node_context,
                                  create_moe_a2a_intra_node_context, gemm_ar_intra_node, gemm_rs_intra_node,
                                  moe_combine_intra_node_op, moe_dispatch_intra_node_op)
    from tridist_b200.utils.testing import fake_expert, moe_inputs
    w = _world1()
    torch.manual_seed(3)
    dt = torch.float16
    M, N, K = 512, 768, 256
    a = (torch.randn(M, K, device="cuda") * 0.05).to(dt)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(dt)
    ref = a.float() @ b.float().t()
    ctx = create_ag_gemm_intra_node_context(M, K, dt, dt, 0, 1, M_PER_CHUNK=256, world=w)
    assert (ag_gemm_intra_node(a, b, False, ctx).float() - ref).abs().max().item() < TOL
    rs = create_gemm_rs_intra_node_context(M, N, dt, 0, 1, world=w)
    assert (gemm_rs_intra_node(a, b, rs).float() - ref).abs().max().item() < TOL
    ar = create_gemm_ar_intra_node_context(M, N, dt, dt, 0, 1, world=w)
    assert (gemm_ar_intra_node(a, b, ar).float() - ref).abs().max().item() < TOL
    E, H, topk, T = 8, 256, 2, 96
    moe = create_moe_a2a_intra_node_context(E, H, dt, T, topk, 0, 1, world=w)
    tokens, idx, wts = [x.cuda() for x in moe_inputs(0, T, H, E, topk, 0, dt)]
    n = int(moe_dispatch_intra_node_op(tokens, idx, moe).item())
    assert n == T * topk
    sc = moe.scatter_idx[:T].long()
    assert sorted(sc.flatten().tolist()) == list(range(n))          # bijection onto rows
    assert torch.equal(moe.recv[sc[:, 0]], tokens)                  # content
    moe.out[:n] = fake_expert(moe.recv[:n])
    out = torch.empty_like(tokens)
    moe_combine_intra_node_op(moe, idx, out, wts)
    exp = (wts.unsqueeze(-1) * (tokens.float().unsqueeze(1) * 2 + (sc % 5).float().unsqueeze(-1))).sum(1)
    torch.cuda.synchronize()
    w.check()
    assert (out.float() - exp).abs().max().item() < 2e-2


def _emu(R):
    from tridist_b200.parallel.runtime import EmulatedWorld
    return EmulatedWorld(R)


@pytest.mark.parametrize("R", [2, 4])
def test_ag_gemm_emulated(R):
    from tridist_b200.ops.all_gather_gemm import ag_gemm_emulated, create_ag_gemm_intra_node_context
    from tridist_b200.utils.testing import ag_inputs
    w = _emu(R)
    dt = torch.bfloat16
    m_pr, K, n_pr = 256, 512, 384
    ctxs = [create_ag_gemm_intra_node_context(m_pr * R, K, dt, dt, r, R, M_PER_CHUNK=128, world=w) for r in range(R)]
    for it in range(3):                                   # fresh data every round, both parities
        ins = [ag_inputs(r, R, m_pr, K, n_pr, it, dt, 0.05) for r in range(R)]
        a_list = [ins[r][0][r].cuda() for r in range(R)]
        b_list = [ins[r][1].cuda() for r in range(R)]
        c_list = [torch.empty(m_pr * R, n_pr, dtype=dt, device="cuda") for _ in range(R)]
        ag_gemm_emulated(ctxs, a_list, b_list, c_list)
        torch.cuda.synchronize()
        w.check()
        full = torch.cat([x.float() for x in a_list], 0)
        for r in range(R):
            ref = full @ b_list[r].float().t()
            assert (c_list[r].float() - ref).abs().max().item() < TOL, f"round {it} rank {r}"
            ws = ctxs[r].workspace(ctxs[r].flag_round & 1, m_pr * R)
            for s in range(R):
                if s != r:                                # pushed shards landed bit-exactly
                    assert torch.equal(ws[s * m_pr:(s + 1) * m_pr], a_list[s])
    # GEMM-only decomposition on the last workspace gives the same result
    c2 = [torch.empty_like(c) for c in c_list]
    ag_gemm_emulated(ctxs, a_list, b_list, c2, skip_comm=True)
    torch.cuda.synchronize()
    for r in range(R):
        assert torch.equal(c2[r], c_list[r])


@pytest.mark.parametrize("R,M", [(2, 512), (4, 512), (4, 256)])
def test_gemm_rs_emulated(R, M):
    from tridist_b200.ops.gemm_reduce_scatter import create_gemm_rs_intra_node_context, gemm_rs_emulated
    from tridist_b200.utils.testing import ks_inputs
    w = _emu(R)
    dt = torch.float16
    N, kl = 384, 256
    ctxs = [create_gemm_rs_intra_node_context(M, N, dt, r, R, world=w) for r in range(R)]
    for it in range(3):
        a_all, b_all = ks_inputs(R, M, N, kl, it, dt, 0.05)
        a_all = [x.cuda() for x in a_all]
        b_all = [x.cuda() for x in b_all]
        outs = gemm_rs_emulated(ctxs, a_all, b_all)
        torch.cuda.synchronize()
        w.check()
        ref = sum(a_all[s].float() @ b_all[s].float().t() for s in range(R))
        m_pr = M // R
        for r in range(R):
            err = (outs[r].float() - ref[r * m_pr:(r + 1) * m_pr]).abs().max().item()
            assert err < TOL, f"round {it} rank {r}: {err}"


@pytest.mark.parametrize("mode", ["one_shot", "two_shot"])
@pytest.mark.parametrize("R,M", [(2, 256), (4, 192)])
def test_gemm_ar_emulated(R, M, mode):
    from tridist_b200.ops.gemm_allreduce import create_gemm_ar_intra_node_context, gemm_ar_emulated
    from tridist_b200.utils.testing import ks_inputs
    w = _emu(R)
    dt = torch.bfloat16
    N, kl = 640, 192
    ctxs = [create_gemm_ar_intra_node_context(256, N, dt, dt, r, R, M_PER_CHUNK=64, world=w) for r in range(R)]
    for it in range(3):
        a_all, b_all = ks_inputs(R, M, N, kl, it, dt, 0.05)
        a_all = [x.cuda() for x in a_all]
        b_all = [x.cuda() for x in b_all]
        use_symm = (mode == "two_shot" and it == 2)
        c_list = [ctxs[r].symm_output(M) if use_symm else torch.empty(M, N, dtype=dt, device="cuda")
                  for r in range(R)]
        gemm_ar_emulated(ctxs, a_all, b_all, c_list, mode=mode)
        torch.cuda.synchronize()
        w.check()
        ref = sum(a_all[s].float() @ b_all[s].float().t() for s in range(R))
        for r in range(R):
            err = (c_list[r].float() - ref).abs().max().item()
            assert err < 2e-2, f"round {it} rank {r}: {err}"
            assert torch.equal(c_list[r], c_list[0]), "all-reduce result must be bit-identical on all ranks"


@pytest.mark.parametrize("zipf", [0.0, 1.2])
def test_moe_emulated(zipf):
    from tridist_b200.ops.moe_a2a import (create_moe_a2a_intra_node_context, moe_combine_emulated,
                                          moe_dispatch_emulated)
    from tridist_b200.utils.testing import fake_expert, moe_inputs
    R, E, H, topk, T = 4, 16, 512, 4, 200
    w = _emu(R)
    dt = torch.float16
    ctxs = [create_moe_a2a_intra_node_context(E, H, dt, T, topk, r, R, world=w) for r in range(R)]
    epr = E // R
    for it in range(2):
        ins = [[x.cuda() for x in moe_inputs(r, T, H, E, topk, it, dt, zipf)] for r in range(R)]
        toks = [i[0] for i in ins]
        idxs = [i[1] for i in ins]
        wts = [i[2] for i in ins]
        totals = moe_dispatch_emulated(ctxs, toks, idxs)
        torch.cuda.synchronize()
        w.check()
        seen = [set() for _ in range(R)]
        for r in range(R):
            n = int(totals[r].item())
            exp_n = sum(int(((idxs[s] // epr) == r).sum()) for s in range(R))
            assert n == exp_n
            # segment layout: (source, local expert) in order, counts match the routing
            counts = ctxs[r].recv_counts.cpu()
            for s in range(R):
                for k in range(epr):
                    assert int(counts[s, k]) == int((idxs[s] == r * epr + k).sum())
        for s in range(R):
            sc = ctxs[s].scatter_idx[:T].cpu()
            ic = idxs[s].cpu()
            for t in range(0, T, 7):
                for j in range(topk):
                    d = int(ic[t, j]) // epr
                    row = int(sc[t, j])
                    assert torch.equal(ctxs[d].recv[row], toks[s][t])            # content
            for t in range(T):
                for j in range(topk):
                    key = (int(ic[t, j]) // epr, int(sc[t, j]))
                    assert key[1] not in seen[key[0]]                               # bijection
                    seen[key[0]].add(key[1])
            # rows of (s -> d, expert) fall inside their segment
        for r in range(R):
            n = int(totals[r].item())
            assert seen[r] == set(range(n))
            ctxs[r].out[:n] = fake_expert(ctxs[r].recv[:n])
        outs = [torch.empty_like(t) for t in toks]
        moe_combine_emulated(ctxs, idxs, outs, wts)
        torch.cuda.synchronize()
        w.check()
        for s in range(R):
            sc = ctxs[s].scatter_idx[:T].long()
            exp = (wts[s].unsqueeze(-1) * (toks[s].float().unsqueeze(1) * 2 + (sc % 5).float().unsqueeze(-1))).sum(1)
            assert (outs[s].float() - exp).abs().max().item() < 3e-2


def test_bounded_wait_reports_status():
    """A wait on a flag nothing sets runs out, records a status and leaves the context usable."""
    from tridist_b200.parallel.runtime import TriDistError
    w = _world1()
    C = _loaded_native()
    w.clear_status()
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    C.wait_flag_test(flag.data_ptr(), 7, w.status_dev, w.abort_word, 50_000_000)   # 50 ms limit
    torch.cuda.synchronize()
    st = w.status()
    assert st[0] == 1 and st[2] == 32 and st[3] == 7 and st[4] == 0
    with pytest.raises(TriDistError):
        w.check()
    w.clear_status()
    w.check()
    # the context still works
    x = torch.ones(8, device="cuda")
    assert float(x.sum()) == 8.0


def test_spot_verify_flags_bad_tile():
    from tridist_b200.ops._gemm_common import gemm_nt
    C = _loaded_native()
    torch.manual_seed(5)
    M, N, K = 256, 512, 256
    a = (torch.randn(M, K, device="cuda") * 0.1).to(torch.float16)
    b = (torch.randn(N, K, device="cuda") * 0.1).to(torch.float16)
    c = gemm_nt(a, b, bn=256)
    bad = torch.zeros(4, dtype=torch.int32, device="cuda")
    C.spot_verify(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, K, K, N, False, 4, 2e-2, bad.data_ptr(), 256)
    torch.cuda.synchronize()
    assert bad.sum().item() == 0
    c[128:, 256:] += 1.0                                  # damage tile (1, 1)
    C.spot_verify(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, K, K, N, False, 4, 2e-2, bad.data_ptr(), 256)
    torch.cuda.synchronize()
    assert bad.tolist() == [0, 0, 0, 1]


def test_skew_layer_order_table_and_observer_emulated():
    """Table-driven source order (device int32 table) gives the same C as the default order, and the
    consumer's arrival stamps come back for every remote source."""
    from tridist_b200.ops.all_gather_gemm import ag_gemm_emulated, create_ag_gemm_intra_node_context
    from tridist_b200.parallel.predictor import infer_straggler
    from tridist_b200.utils.testing import ag_inputs
    R = 4
    w = _emu(R)
    dt = torch.float16
    m_pr, K, n_pr = 128, 256, 256
    ctxs = [create_ag_gemm_intra_node_context(m_pr * R, K, dt, dt, r, R, M_PER_CHUNK=128, world=w) for r in range(R)]
    ins = [ag_inputs(r, R, m_pr, K, n_pr, 0, dt, 0.05) for r in range(R)]
    a_list = [ins[r][0][r].cuda() for r in range(R)]
    b_list = [ins[r][1].cuda() for r in range(R)]
    c_ref = [torch.empty(m_pr * R, n_pr, dtype=dt, device="cuda") for _ in range(R)]
    ag_gemm_emulated(ctxs, a_list, b_list, c_ref)
    torch.cuda.synchronize()
    for r, ctx in enumerate(ctxs):                         # own first, "straggler" (r+1) last
        order = [r] + [x for x in range(R) if x not in (r, (r + 1) % R)] + [(r + 1) % R]
        ctx.emu_order_table = torch.tensor(order, dtype=torch.int32, device="cuda")
        ctx.observe = True
        ctx.arrival_ns.fill_(torch.iinfo(torch.int64).max)
    c_tab = [torch.empty_like(c) for c in c_ref]
    ag_gemm_emulated(ctxs, a_list, b_list, c_tab)
    torch.cuda.synchronize()
    w.check()
    for r in range(R):
        assert torch.equal(c_tab[r], c_ref[r])
        stamps = ctxs[r].arrival_ns.cpu().tolist()
        remote = [s for s in range(R) if s != r]
        assert all(0 < stamps[s] < torch.iinfo(torch.int64).max for s in remote)
        assert infer_straggler(stamps, r) in remote


def test_verify_and_repair_single_rank(monkeypatch):
    from tridist_b200.ops import create_i1_context, i1_ag_tr_op, i1_observer_read, i1_table_peek, i1_table_write
    from tridist_b200.ops.ag_tr_pred import _verify_and_repair
    w = _world1()
    dt = torch.bfloat16
    M, K, N = 512, 256, 512
    torch.manual_seed(11)
    a = (torch.randn(M, K, device="cuda") * 0.1).to(dt)
    b = (torch.randn(N, K, device="cuda") * 0.1).to(dt)
    c = torch.empty(M, N, dtype=dt, device="cuda")
    ictx = create_i1_context(M, K, dt, dt, 0, 1, world=w)
    i1_table_write(ictx, 7, 0, 1, 0, 1)
    assert i1_table_peek(ictx)[:4] == [7, 0, 1, 1]
    i1_ag_tr_op(a, b, c, ictx)
    torch.cuda.synchronize()
    good = c.clone()
    assert (good.float() - a.float() @ b.float().t()).abs().max().item() < TOL
    assert _verify_and_repair(a, b, c, ictx) == 0         # nothing to repair
    c[128:256, 256:] = 0                                  # damage one tile of the result
    fixed = _verify_and_repair(a, b, c, ictx)
    torch.cuda.synchronize()
    assert fixed >= 1 and torch.equal(c, good)
    assert i1_observer_read(ictx)[1] == 0


def test_order_driven_ar_carrier_and_gates_single_rank():
    from tridist_b200.ops import (create_gemm_ar_rd_context, gemm_ar_pred_op, make_gate_flag, task_events)
    w = _world1()
    dt = torch.float16
    M, N, K = 256, 256, 128
    torch.manual_seed(12)
    a = (torch.randn(M, K, device="cuda") * 0.1).to(dt)
    b = (torch.randn(N, K, device="cuda") * 0.1).to(dt)
    ctx = create_gemm_ar_rd_context(M, N, dt, dt, 0, 1, world=w)
    ctx.chunk_rows = 64
    gate = make_gate_flag()
    gate[0] = 5                                           # already released
    c = torch.zeros(M, N, dtype=dt, device="cuda")
    gemm_ar_pred_op(a, b, c, ctx, order=[3, 1, 0, 2], gates=[(1, gate.data_ptr(), 5)])
    torch.cuda.synchronize()
    w.check()
    assert (c.float() - a.float() @ b.float().t()).abs().max().item() < TOL
    ev = task_events(ctx)
    assert len(ev) == 4 and all(e is not None and e[0].elapsed_time(e[1]) >= 0 for e in ev)


def test_symm_host_one_sided_calls():
    from tridist_b200.parallel.symm_host import SymmHost
    w = _world1()
    h = SymmHost(w)
    assert h.my_pe() == 0 and h.n_pes() == 1
    buf = h.malloc(4096)
    src = torch.arange(256, dtype=torch.int32, device="cuda")
    h.putmem(buf, 1024, src, pe=0)
    dst = torch.zeros_like(src)
    h.getmem(dst, buf, 1024, pe=0)
    h.quiet()
    assert torch.equal(src, dst) and h.ptr(buf, 0, 16) == buf.local_ptr + 16
    h.set_signal(buf, 3, 9, pe=0)
    h.wait_signal(buf, 3, 9, timeout_ms=200)
    h.barrier_all()
    torch.cuda.synchronize()
    w.check()
    h.free(buf)


@pytest.mark.parametrize("mode", ["ag_rs", "gemm_ar"])
def test_tp_mlp_single_rank(mode):
    from tridist_b200.models.tp_mlp import TPMLP, TPMLPConfig, reference_forward
    w = _world1()
    dt = torch.bfloat16
    M, K, I = 256, 256, 384
    torch.manual_seed(13)
    x = torch.randn(M, K, device="cuda").to(dt)
    w_gu = (torch.randn(2 * I, K, device="cuda") * 0.05).to(dt)
    w_d = (torch.randn(K, I, device="cuda") * 0.05).to(dt)
    ref = reference_forward(x, [w_gu], [w_d])
    for fuse in ([True, False] if mode == "ag_rs" else [False]):
        layer = TPMLP(TPMLPConfig(hidden=K, intermediate=I, max_tokens=M, dtype=dt, mode=mode, fuse_swiglu=fuse),
                      0, 1, w_gu, w_d, world=w)
        y = layer(x)
        torch.cuda.synchronize()
        w.check()
        assert (y.float() - ref).abs().max().item() < 3e-2


# ---------------------------------------------------------------------------------------------
# The persistent loop, the tile shapes and the edges (every CTA gets many tiles: accumulator
# reuse, ring wrap across tiles, late-joining pushers; odd block counts; ragged M and N)
# ---------------------------------------------------------------------------------------------
def _rand(shape, seed, dtype, scale=0.05):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(dtype)


def _check_rows(out, a, b, rows=96, tol=TOL):
    idx = torch.randperm(a.shape[0], device="cuda")[:rows]
    ref = a[idx].float() @ b.float().t()
    err = (out[idx].float() - ref).abs().max().item()
    assert err < tol, err


@pytest.mark.parametrize("variant", ["wide", "pair", "single"])
@pytest.mark.parametrize("K", [2048, 12288])
def test_plain_gemm_many_tiles_per_cta(variant, K, monkeypatch):
    """16 CTAs for 4096 x 4096: every CTA (pair) walks 16 to 64 tiles, so both accumulators are
    reused many times and the operand ring wraps across tile boundaries."""
    from tridist_b200.ops._gemm_common import gemm_nt
    monkeypatch.setenv("TRIDIST_WIDE", "1" if variant == "wide" else "0")
    monkeypatch.setenv("TRIDIST_CTA_PAIR", "0" if variant == "single" else "1")
    a, b = _rand((4096, K), 21, torch.bfloat16), _rand((4096, K), 22, torch.bfloat16)
    out = gemm_nt(a, b, max_ctas=16)
    torch.cuda.synchronize()
    _check_rows(out, a, b)


@pytest.mark.parametrize("splitk", [1, 0])
@pytest.mark.parametrize("M,N,K,max_ctas", [(128, 2048, 4096, 0), (128, 1024, 8200, 0), (1536, 1024, 2048, 10),
                                            (2048, 2304, 1024, 20), (640, 648, 1024, 0), (1000, 520, 776, 0),
                                            (384, 768, 512, 0), (4224, 512, 256, 12)])
def test_plain_gemm_edges_and_split_k(M, N, K, max_ctas, splitk, monkeypatch):
    """Ragged M / N / K, odd numbers of row blocks under CTA pairs and 512-row tiles, and the K
    split of the last scheduling round (2 to 8 slices; K blocks that do not divide evenly)."""
    from tridist_b200.ops._gemm_common import gemm_nt
    monkeypatch.setenv("TRIDIST_SPLITK", str(splitk))
    for dt in (torch.float16, torch.bfloat16):
        a, b = _rand((M, K), 31, dt), _rand((N, K), 32, dt)
        out = gemm_nt(a, b, max_ctas=max_ctas)
        torch.cuda.synchronize()
        ref = a.float() @ b.float().t()
        assert (out.float() - ref).abs().max().item() < TOL


def test_split_k_slices_are_used(monkeypatch):
    from tridist_b200.ops._gemm_common import BM, OP_PLAIN, SCHED_NATURAL
    C = _loaded_native()
    for M, N, K in [(128, 2048, 4096), (128, 8192, 3584), (8192, 6144, 12288)]:
        cuts = C.splitk_dump(dict(op=OP_PLAIN, sched=SCHED_NATURAL, bn=256 if M > 128 else 128, R=1, rank=0,
                                  M=M, N=N, K=K), 148)
        assert cuts and all(2 <= c[3] <= 8 for c in cuts)


@pytest.mark.parametrize("tiles", ["single", "pair", "wide"])
def test_fused_ops_emulated_many_tiles_per_cta(tiles, monkeypatch):
    """Two virtual ranks, 8 CTAs each, 2048-row problems: AG (pushing CTAs join late), RS and both
    AR forms walk many tiles per CTA, on single CTAs, CTA pairs and 512-row pair tiles."""
    from tridist_b200.ops.all_gather_gemm import ag_gemm_emulated, create_ag_gemm_intra_node_context
    from tridist_b200.ops.gemm_allreduce import create_gemm_ar_intra_node_context, gemm_ar_emulated
    from tridist_b200.ops.gemm_reduce_scatter import create_gemm_rs_intra_node_context, gemm_rs_emulated
    monkeypatch.setenv("TRIDIST_MAX_CTAS", "8")
    monkeypatch.setenv("TRIDIST_EMU_PAIR", "0" if tiles == "single" else "1")
    monkeypatch.setenv("TRIDIST_WIDE", "1" if tiles == "wide" else "0")
    monkeypatch.setenv("TRIDIST_PUSH_CTAS", "4")
    monkeypatch.setenv("TRIDIST_PUSH_SKIP", "1")
    R, dt = 2, torch.bfloat16
    w = _emu(R)
    M, N, K = 2048, 1024, 768
    m_pr = M // R
    ag = [create_ag_gemm_intra_node_context(M, K, dt, dt, r, R, M_PER_CHUNK=512, world=w) for r in range(R)]
    rs = [create_gemm_rs_intra_node_context(M, N, dt, r, R, world=w) for r in range(R)]
    ar = [create_gemm_ar_intra_node_context(M, N, dt, dt, r, R, M_PER_CHUNK=64, world=w) for r in range(R)]
    for it in range(2):
        a_sh = [_rand((m_pr, K), 40 + 7 * it + r, dt) for r in range(R)]
        bw = [_rand((N, K), 50 + 7 * it + r, dt) for r in range(R)]
        c = [torch.empty(M, N, dtype=dt, device="cuda") for _ in range(R)]
        ag_gemm_emulated(ag, a_sh, bw, c)
        torch.cuda.synchronize()
        w.check()
        full = torch.cat(a_sh, 0)
        for r in range(R):
            _check_rows(c[r], full, bw[r])
        a_k = [_rand((M, K), 60 + 7 * it + r, dt) for r in range(R)]
        ref = sum(a_k[s].float() @ bw[s].float().t() for s in range(R))
        outs = gemm_rs_emulated(rs, a_k, bw)
        torch.cuda.synchronize()
        w.check()
        for r in range(R):
            assert (outs[r].float() - ref[r * m_pr:(r + 1) * m_pr]).abs().max().item() < 2e-2
        for mode in ("one_shot", "two_shot"):
            cc = [torch.empty(M, N, dtype=dt, device="cuda") for _ in range(R)]
            gemm_ar_emulated(ar, a_k, bw, cc, mode=mode)
            torch.cuda.synchronize()
            w.check()
            for r in range(R):
                assert (cc[r].float() - ref).abs().max().item() < 2e-2, mode
                assert torch.equal(cc[r], cc[0])


@pytest.mark.parametrize("R,M", [(4, 768), (2, 384), (4, 1280)])
def test_gemm_rs_emulated_rows_per_rank_not_a_block_multiple(R, M):
    """Rows per rank of 192 / 320: row blocks with two owners take the per-row bulk path, and two
    owners of one block publish before either waits."""
    from tridist_b200.ops.gemm_reduce_scatter import create_gemm_rs_intra_node_context, gemm_rs_emulated
    w = _emu(R)
    dt = torch.float16
    N, kl = 640, 320
    ctxs = [create_gemm_rs_intra_node_context(M, N, dt, r, R, world=w) for r in range(R)]
    for it in range(2):
        a_all = [_rand((M, kl), 70 + it * 9 + r, dt) for r in range(R)]
        b_all = [_rand((N, kl), 80 + it * 9 + r, dt) for r in range(R)]
        outs = gemm_rs_emulated(ctxs, a_all, b_all)
        torch.cuda.synchronize()
        w.check()
        ref = sum(a_all[s].float() @ b_all[s].float().t() for s in range(R))
        m_pr = M // R
        for r in range(R):
            assert (outs[r].float() - ref[r * m_pr:(r + 1) * m_pr]).abs().max().item() < TOL


def test_fused_kernel_gives_up_cleanly_when_a_shard_never_arrives(monkeypatch):
    """The allowed form of a failure test: virtual rank 1 does not push, rank 0's producer waits
    for its shard with a 20 ms limit, the wait runs out, every role of the kernel unwinds (loads
    drained, MMAs retired, TMEM freed), the status names the site, and the next launch on the same
    context works."""
    from tridist_b200.ops.all_gather_gemm import ag_gemm_emulated, create_ag_gemm_intra_node_context
    from tridist_b200.parallel.runtime import TriDistError
    monkeypatch.setenv("TRIDIST_WAIT_TIMEOUT_MS", "20")
    R, dt = 2, torch.float16
    w = _emu(R)
    m_pr, K, N = 256, 512, 512
    ctxs = [create_ag_gemm_intra_node_context(m_pr * R, K, dt, dt, r, R, M_PER_CHUNK=128, world=w) for r in range(R)]
    a = [_rand((m_pr, K), 90 + r, dt) for r in range(R)]
    b = [_rand((N, K), 95 + r, dt) for r in range(R)]
    c = [torch.empty(m_pr * R, N, dtype=dt, device="cuda") for _ in range(R)]
    ag_gemm_emulated(ctxs, a, b, c)                      # a good round first
    torch.cuda.synchronize()
    w.check()
    ag_gemm_emulated(ctxs, a, b, c, mute_ranks=[1])      # rank 1's shard never arrives at rank 0
    torch.cuda.synchronize()
    with pytest.raises(TriDistError, match="all-gather chunk ticket"):
        w.check()
    st = w.status()
    assert st[0] == 1 and st[1] == 0 and st[2] == 1      # flag wait timed out, on rank 0, at the chunk ticket
    w.clear_status()
    ag_gemm_emulated(ctxs, a, b, c)                      # the context is still usable
    torch.cuda.synchronize()
    w.check()
    full = torch.cat(a, 0).float()
    for r in range(R):
        assert (c[r].float() - full @ b[r].float().t()).abs().max().item() < TOL


def test_a_rank_that_gives_up_raises_every_ranks_abort_word():
    """The abort buffer is symmetric: the kernel that runs out of time stores its code into the abort
    word of every rank, and a kernel that leaves a wait because of a raised word records why."""
    w = _emu(3)
    C = _loaded_native()
    w.clear_status()
    words = w.peer_abort_words()
    assert len(set(words)) == 3
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    C.wait_flag_test(flag.data_ptr(), 9, w.status_dev, words[0], 20_000_000, words)
    torch.cuda.synchronize()
    raised = [int(w.abort_buf.tensor(torch.int32, (1,), 0, rank=r).item()) for r in range(3)]
    assert raised == [1, 1, 1]
    assert w.status()[0] == 1
    # a second waiter whose word is already raised leaves at once and records "gave up because ..."
    from tridist_b200.parallel.runtime import TriDistError
    w.C.status_clear(w.status_host)
    C.wait_flag_test(flag.data_ptr(), 9, w.status_dev, words[1], 2_000_000_000, [])
    torch.cuda.synchronize()
    assert w.status()[0] == 5
    with pytest.raises(TriDistError, match="another rank"):
        w.check()
    w.clear_status()
    assert [int(w.abort_buf.tensor(torch.int32, (1,), 0, rank=r).item()) for r in range(3)] == [0, 0, 0]


@pytest.mark.parametrize("R", [2, 4])
def test_ag_gemm_pull_transport_emulated(R):
    """The tile-ready entry points: stage, arrive tickets, pull through the copy engine, ready tickets."""
    from tridist_b200.ops.all_gather_gemm import ag_gemm_emulated
    from tridist_b200.ops.gemm_ag_tr import create_gemm_ag_tr_context
    w = _emu(R)
    dt = torch.float16
    m_pr, K, n_pr = 256, 1024, 384
    ctxs = [create_gemm_ag_tr_context(m_pr * R, K, dt, dt, r, R, chunk_rows=128, world=w) for r in range(R)]
    assert all(c.transport == "pull" for c in ctxs)
    for it in range(3):
        a = [_rand((m_pr, K), 200 + it * 5 + r, dt) for r in range(R)]
        b = [_rand((n_pr, K), 210 + it * 5 + r, dt) for r in range(R)]
        c = [torch.empty(m_pr * R, n_pr, dtype=dt, device="cuda") for _ in range(R)]
        ag_gemm_emulated(ctxs, a, b, c)
        torch.cuda.synchronize()
        w.check()
        full = torch.cat(a, 0).float()
        for r in range(R):
            assert (c[r].float() - full @ b[r].float().t()).abs().max().item() < TOL, f"round {it} rank {r}"
            ws = ctxs[r].workspace(ctxs[r].flag_round & 1, m_pr * R)
            for s in range(R):                      # own shard staged, the others pulled, all bit-exact
                assert torch.equal(ws[s * m_pr:(s + 1) * m_pr], a[s])


def test_skew_table_modes_give_the_same_result_emulated():
    """The full table [seq, degraded, mode, k_eff, order[R], budget[R]] read by the kernel: band-major
    (mode 0, two row bands), source-major (mode 1), degraded (default rotation) and small spin budgets
    only change which CTA computes which tile when."""
    from tridist_b200.ops.all_gather_gemm import ag_gemm_emulated, create_ag_gemm_intra_node_context
    R = 4
    w = _emu(R)
    dt = torch.bfloat16
    m_pr, K, n_pr = 512, 512, 512
    ctxs = [create_ag_gemm_intra_node_context(m_pr * R, K, dt, dt, r, R, M_PER_CHUNK=256, world=w) for r in range(R)]
    a = [_rand((m_pr, K), 300 + r, dt) for r in range(R)]
    b = [_rand((n_pr, K), 310 + r, dt) for r in range(R)]
    ref = [torch.empty(m_pr * R, n_pr, dtype=dt, device="cuda") for _ in range(R)]
    ag_gemm_emulated(ctxs, a, b, ref)
    torch.cuda.synchronize()
    w.check()
    full = torch.cat(a, 0).float()
    assert (ref[0].float() - full @ b[0].float().t()).abs().max().item() < 2e-2
    for seq, (deg, mode, k_eff, budget) in enumerate([(0, 0, 2, 128), (0, 1, 2, 128), (1, 1, 2, 128), (0, 0, 2, 1)]):
        tables = []
        for r, ctx in enumerate(ctxs):
            order = [r] + [x for x in range(R) if x not in (r, (r + 1) % R)] + [(r + 1) % R]
            t = torch.tensor([seq, deg, mode, k_eff] + order + [budget] * R, dtype=torch.int32, device="cuda")
            tables.append(t)
            ctx.emu_order_table = t[4:4 + R]
            ctx.emu_table_header = True
            ctx.plans.clear()
        out = [torch.empty_like(x) for x in ref]
        ag_gemm_emulated(ctxs, a, b, out)
        torch.cuda.synchronize()
        w.check()
        for r in range(R):
            assert torch.equal(out[r], ref[r]), (deg, mode, k_eff, budget, r)


def test_band_major_schedule_walks_bands_first():
    C = _loaded_native()
    from tridist_b200.ops._gemm_common import OP_AG, SCHED_SEGMENT
    R, M, N = 4, 4096, 1024
    d = dict(op=OP_AG, sched=SCHED_SEGMENT, bn=256, R=R, rank=1, M=M, N=N, K=1024, m_per_rank=M // R,
             seg_order=[1, 0, 3, 2], chunk_rows=256, n_chunks=4, seg_bands=2, allow_wide=0)
    tiles = sorted((t[4], t[0]) for cta in C.schedule_dump(d, 148) for t in cta)
    rows_per_seg = (M // R) // 128
    walk = []
    for _, mt in tiles:
        key = (mt // rows_per_seg, (mt % rows_per_seg) // (rows_per_seg // 2))     # (segment, band)
        if not walk or walk[-1] != key:
            walk.append(key)
    assert walk == [(s, b) for b in range(2) for s in [1, 0, 3, 2]]


def test_device_side_index_check_reports_and_skips():
    """A row index outside the receive buffer (made here by damaging the scatter table between dispatch
    and combine) is recorded as 'index out of range' and the access is skipped: nothing faults."""
    from tridist_b200.ops import (create_moe_a2a_intra_node_context, moe_combine_intra_node_op,
                                  moe_dispatch_intra_node_op)
    from tridist_b200.parallel.runtime import TriDistError
    from tridist_b200.utils.testing import moe_inputs
    w = _world1()
    w.clear_status()
    dt = torch.float16
    E, H, topk, T = 8, 256, 2, 64
    ctx = create_moe_a2a_intra_node_context(E, H, dt, T, topk, 0, 1, world=w)
    tokens, idx, wts = [x.cuda() for x in moe_inputs(0, T, H, E, topk, 3, dt)]
    moe_dispatch_intra_node_op(tokens, idx, ctx)
    ctx.out[:T * topk] = ctx.recv[:T * topk]
    ctx.scatter_idx[5, 1] = ctx.recv.shape[0] + 17
    out = torch.empty_like(tokens)
    moe_combine_intra_node_op(ctx, idx, out, wts)
    torch.cuda.synchronize()
    st = w.status()
    assert st[0] == 3 and st[2] == 11 and st[4] == ctx.recv.shape[0] + 17
    with pytest.raises(TriDistError, match="index out of range"):
        w.check()
    w.clear_status()
    assert bool(torch.isfinite(out.float()).all())


@pytest.mark.parametrize("R", [2, 4, 8])
def test_gemm_ar_rd_emulated(R):
    """Recursive-doubling panel exchange on virtual ranks: three panels over two staging slots (the
    third panel reuses slot 0 under the ack ticket), several calls on one context, and an M that
    changes between calls (tickets advance by a fixed stride per call)."""
    from tridist_b200.ops.gemm_ar_rd import create_gemm_ar_rd_context, gemm_ar_rd_emulated
    from tridist_b200.utils.testing import ks_inputs
    w = _emu(R)
    dt = torch.bfloat16
    N, kl = 640, 192
    ctxs = [create_gemm_ar_rd_context(384, N, dt, dt, r, R, chunk_rows=128, stage_slots=2, world=w)
            for r in range(R)]
    assert ctxs[0].rd.num_chunks == 3 and ctxs[0].rd.phases == R.bit_length() - 1
    for it, M in enumerate((384, 256, 384, 128)):
        a_all, b_all = ks_inputs(R, M, N, kl, it, dt, 0.05)
        a_all = [x.cuda() for x in a_all]
        b_all = [x.cuda() for x in b_all]
        c_list = [torch.empty(M, N, dtype=dt, device="cuda") for _ in range(R)]
        gemm_ar_rd_emulated(ctxs, a_all, b_all, c_list)
        torch.cuda.synchronize()
        w.check()
        ref = sum(a_all[s].float() @ b_all[s].float().t() for s in range(R))
        for r in range(R):
            err = (c_list[r].float() - ref).abs().max().item()
            assert err < 3e-2, f"call {it} rank {r}: {err}"
            assert torch.equal(c_list[r], c_list[0]), "all ranks must hold bit-identical results"


def test_gemm_ar_rd_ack_wait_runs_out():
    """A staging slot whose previous occupant is never acknowledged: the exchange kernel's wait
    runs out (20 ms limit), the kernel returns with a status record naming the ack ticket, the
    other virtual rank leaves through the abort word, and the context stays usable."""
    from tridist_b200.ops.gemm_ar_rd import create_gemm_ar_rd_context, gemm_ar_rd_emulated
    from tridist_b200.parallel.runtime import TriDistError
    from tridist_b200.utils.testing import ks_inputs
    R, M, N, kl = 2, 128, 256, 64
    w = _emu(R)
    w.timeout_ms = 20
    dt = torch.float16
    ctxs = [create_gemm_ar_rd_context(M, N, dt, dt, r, R, chunk_rows=128, stage_slots=1, world=w) for r in range(R)]
    a_all, b_all = [[x.cuda() for x in xs] for xs in ks_inputs(R, M, N, kl, 0, dt, 0.05)]
    c_list = [torch.empty(M, N, dtype=dt, device="cuda") for _ in range(R)]
    ctxs[1].rd.last_ticket_per_slot[0] = 1 << 19          # an occupant nobody will ever acknowledge
    gemm_ar_rd_emulated(ctxs, a_all, b_all, c_list)
    torch.cuda.synchronize()
    with pytest.raises(TriDistError, match="recursive-doubling ack ticket"):
        w.check()
    w.clear_status()
    for ctx in ctxs:                                       # forget the poisoned slot; tickets only grow
        ctx.rd.last_ticket_per_slot[0] = 0
    gemm_ar_rd_emulated(ctxs, a_all, b_all, c_list)
    torch.cuda.synchronize()
    w.check()
    ref = sum(a_all[s].float() @ b_all[s].float().t() for s in range(R))
    assert (c_list[0].float() - ref).abs().max().item() < 2e-2 and torch.equal(c_list[0], c_list[1])


def test_own_first_band_walk_emulated():
    """The walk the multicast all-gather uses (own rows, then row unit b of every other source before
    unit b + 1 of any) on virtual ranks with the bulk-copy push: only the order of the tiles changes,
    the result is bit-identical to the source-major walk."""
    from tridist_b200.ops.all_gather_gemm import ag_gemm_emulated, create_ag_gemm_intra_node_context
    R = 4
    w = _emu(R)
    dt = torch.bfloat16
    m_pr, K, n_pr = 1024, 256, 512
    ctxs = [create_ag_gemm_intra_node_context(m_pr * R, K, dt, dt, r, R, M_PER_CHUNK=256, world=w) for r in range(R)]
    a = [_rand((m_pr, K), 700 + r, dt) for r in range(R)]
    b = [_rand((n_pr, K), 710 + r, dt) for r in range(R)]
    ref = [torch.empty(m_pr * R, n_pr, dtype=dt, device="cuda") for _ in range(R)]
    ag_gemm_emulated(ctxs, a, b, ref)
    torch.cuda.synchronize()
    w.check()
    assert (ref[1].float() - torch.cat(a, 0).float() @ b[1].float().t()).abs().max().item() < 2e-2
    for ctx in ctxs:
        ctx.seg_bands, ctx.seg_own_first = -1, 1
        ctx.plans.clear()
    for it in range(2):                              # both workspace parities
        out = [torch.empty_like(x) for x in ref]
        ag_gemm_emulated(ctxs, a, b, out)
        torch.cuda.synchronize()
        w.check()
        for r in range(R):
            assert torch.equal(out[r], ref[r]), (it, r)
