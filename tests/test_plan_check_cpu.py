"""The host-side bounds check of a GEMM plan (TRIDIST_DEBUG=1 runs it before every plan creation):
consistent descriptions pass, an undersized buffer or ticket plane is named."""
import pytest

from tridist_b200.ops._gemm_common import (OP_AG, OP_AR1, OP_AR2, OP_PLAIN, OP_RS, SCHED_NATURAL, SCHED_SEGMENT,
                                           SCHED_STRIDED, rotation_order)


def _check(d, **ext):
    from tridist_b200.parallel.runtime import native
    base = dict(op=OP_PLAIN, sched=SCHED_NATURAL, bn=256, R=1, rank=0, K=4096)
    base.update(d)
    base.setdefault("ldc", base["N"])
    return native().plan_check(base, ext, 148)


def test_plain():
    M, N = 4096, 6144
    assert _check(dict(M=M, N=N), c_bytes=M * N * 2) == []
    bad = _check(dict(M=M, N=N), c_bytes=M * N * 2 - 2)
    assert len(bad) == 1 and bad[0].startswith("output c needs")
    # a strided output (ldc > N) needs the longer extent
    assert _check(dict(M=M, N=N, ldc=N + 64), c_bytes=M * N * 2) != []
    assert _check(dict(M=M, N=N, ldc=N + 64), c_bytes=((M - 1) * (N + 64) + N) * 2) == []


@pytest.mark.parametrize("R", [2, 8])
def test_all_gather(R):
    M, N, K, rank = 8192, 6144, 4096, 1
    m_pr = M // R
    d = dict(op=OP_AG, sched=SCHED_SEGMENT, M=M, N=N, K=K, R=R, rank=rank, m_per_rank=m_pr,
             seg_order=rotation_order(rank, R, 1, own_last=False), chunk_rows=m_pr // 2, n_chunks=2,
             push_ctas=32, push_skip_rounds=1)
    good = dict(c_bytes=M * N * 2, ws_bytes=M * K * 2, ag_flag_words=R * 2)
    assert _check(d, **good) == []
    assert any("workspace" in s for s in _check(d, **dict(good, ws_bytes=M * K * 2 - 16)))
    assert any("ticket plane" in s for s in _check(d, **dict(good, ag_flag_words=R * 2 - 1)))
    assert any("chunk_rows" in s for s in _check(dict(d, n_chunks=3), **good))


@pytest.mark.parametrize("R", [2, 8])
def test_reduce_scatter(R):
    M, N, rank = 8192, 12288, R - 1
    m_pr = M // R
    d = dict(op=OP_RS, sched=SCHED_SEGMENT, M=M, N=N, R=R, rank=rank, m_per_rank=m_pr, slot_stride=m_pr * N,
             seg_order=rotation_order(rank, R, 1, own_last=True))
    tiles = (M // 128) * (N // 256)
    good = dict(c_bytes=m_pr * N * 2, slot_bytes=M * N * 2, tile_flag_words=R * tiles)
    assert _check(d, **good) == []
    assert any("partial slots" in s for s in _check(d, **dict(good, slot_bytes=M * N * 2 - 2)))
    assert any("tile ticket plane" in s for s in _check(d, **dict(good, tile_flag_words=R * tiles - 1)))
    assert any("slot stride" in s for s in _check(dict(d, slot_stride=m_pr * N - 8), **good))
    assert any("output c" in s for s in _check(d, **dict(good, c_bytes=m_pr * N * 2 - 2)))


@pytest.mark.parametrize("mode", ["one_shot", "two_shot", "nvls"])
def test_all_reduce(mode):
    R, rank, M, N = 8, 2, 4096, 8192
    plane = M * N
    d = dict(M=M, N=N, R=R, rank=rank, slot_stride=plane)
    if mode == "one_shot":
        d.update(op=OP_AR1)
        tickets = (M // 128) * (N // 256)
    else:
        d.update(op=OP_AR2, sched=SCHED_STRIDED, strided_interleave=1,
                 seg_order=rotation_order(rank, R, 1, own_last=True))
        tickets = (M // 256) * 2 * (N // 256)
    if mode == "nvls":
        d.update(nvls=1, slot_stride=0, mc_part=[1 << 40, (1 << 40) + 2 * plane], mc_res=[1 << 41, (1 << 41) + 2 * plane])
    good = dict(c_bytes=plane * 2, slot_bytes=(plane if mode == "nvls" else R * plane) * 2, tile_flag_words=R * tickets)
    if mode != "one_shot":
        good.update(res_bytes=plane * 2, res_flag_words=R * tickets)      # result tickets: one row per owner
    assert _check(d, **good) == []
    assert _check(d, **dict(good, slot_bytes=good["slot_bytes"] - 2)) != []
    assert _check(d, **dict(good, tile_flag_words=R * tickets - 1)) != []
    if mode != "one_shot":
        assert any("result plane" in s for s in _check(d, **dict(good, res_bytes=plane * 2 - 2)))
        assert any("result ticket plane" in s for s in _check(d, **dict(good, res_flag_words=R * tickets - 1)))
        # a context-wide stride larger than this call's ticket count widens both planes
        wide = dict(d, ticket_stride=2 * tickets)
        assert _check(wide, **good) != []
        assert _check(wide, **dict(good, tile_flag_words=(R - 1) * 2 * tickets + tickets,
                                   res_flag_words=(R - 1) * 2 * tickets + tickets)) == []


def test_unknown_extents_are_skipped():
    assert _check(dict(M=1024, N=1024)) == []


def test_random_shapes_schedule_is_consistent():
    """300 pseudo-random (operator, shape, ranks, tile width, pairing, push) combinations: every tile
    once, ticket indices unique and in range (odd numbers of row blocks with CTA pairs included)."""
    import random
    rnd = random.Random(7)
    checked = 0
    while checked < 300:
        R = rnd.choice([1, 2, 4, 8])
        op = rnd.choice([OP_PLAIN, OP_AG, OP_RS, OP_AR1, OP_AR2]) if R > 1 else OP_PLAIN
        rank = rnd.randrange(R)
        if op in (OP_AG, OP_RS):
            m_pr = rnd.choice([128, 256, 384, 512, 1024, 1152]) if op == OP_AG else rnd.choice([64, 128, 256, 384, 1152])
            M = m_pr * R
            if M % 128:
                continue
        else:
            M = rnd.choice([64, 128, 192, 256, 384, 1024, 4096, 4224])
            m_pr = M
        N = rnd.choice([128, 256, 384, 768, 1024, 2048, 8192, 6272])
        d = dict(op=op, bn=rnd.choice([128, 256]), R=R, rank=rank, M=M, N=N, K=1024, allow_pair=rnd.choice([0, 1]))
        if op == OP_AG:
            d.update(sched=SCHED_SEGMENT, m_per_rank=m_pr, seg_order=rotation_order(rank, R, 1, own_last=False),
                     chunk_rows=m_pr, n_chunks=1, push_ctas=rnd.choice([0, 8, 32]), push_skip_rounds=rnd.choice([0, 1, 2]))
        elif op == OP_RS:
            d.update(sched=SCHED_SEGMENT if m_pr % 128 == 0 else SCHED_NATURAL, m_per_rank=m_pr,
                     seg_order=rotation_order(rank, R, 1, own_last=True), slot_stride=m_pr * N)
        elif op == OP_AR2:
            d.update(sched=SCHED_STRIDED, seg_order=rotation_order(rank, R, 1, own_last=True),
                     strided_interleave=rnd.choice([0, 1]), slot_stride=M * N)
        elif op == OP_AR1:
            d.update(slot_stride=M * N)
        assert _check(d) == [], d
        checked += 1
