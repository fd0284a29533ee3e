"""The fused GEMM kernel's tile schedule, replayed on the host (the same C++ functions the
device code runs): every output tile is computed exactly once, tickets are unique, owners of
the two-shot all-reduce are balanced, segment orders are honoured and the CTAs that push the
all-gather shard join late. Needs the built extension but no GPU."""
import itertools

import pytest

from tridist_b200.ops._gemm_common import (OP_AG, OP_AR2, OP_PLAIN, OP_RS, SCHED_NATURAL, SCHED_SEGMENT,
                                           SCHED_STRIDED, rotation_order)

BM = 128


def _dump(**kw):
    from tridist_b200.parallel.runtime import native
    d = dict(op=OP_PLAIN, sched=SCHED_NATURAL, bn=256, R=1, rank=0, K=4096)
    d.update(kw)
    return native().schedule_dump(d, 148)


def _tiles(M, N, bn):
    return set(itertools.product(range((M + BM - 1) // BM), range((N + bn - 1) // bn)))


@pytest.mark.parametrize("M,N,bn,pair", [(8192, 6144, 256, 1), (8192, 6144, 256, 0), (1024, 8192, 128, 1),
                                         (128, 8192, 128, 1), (384, 768, 256, 1), (4096 + 128, 2048, 256, 1)])
def test_plain_covers_every_tile_once(M, N, bn, pair):
    out = _dump(M=M, N=N, bn=bn, allow_pair=pair)
    seen = [(t[0], t[1]) for cta in out for t in cta if t[0] * BM < M]
    assert len(seen) == len(set(seen))
    assert set(seen) == _tiles(M, N, bn)
    tickets = [t[2] for cta in out for t in cta]
    assert len(tickets) == len(set(tickets))
    assert len(out) <= 148


def test_pairs_take_adjacent_row_blocks():
    out = _dump(M=8192, N=6144, bn=256)
    for even, odd in zip(out[0::2], out[1::2]):
        assert [(t[0] + 1, t[1]) for t in even] == [(t[0], t[1]) for t in odd]
        assert all(t[0] % 2 == 0 for t in even)


@pytest.mark.parametrize("R", [2, 4, 8])
def test_allgather_segments_and_late_pushers(R):
    M, N, rank = 8192, 6144, 1
    order = rotation_order(rank, R, 1, own_last=False)
    kw = dict(op=OP_AG, sched=SCHED_SEGMENT, M=M, N=N, bn=256, R=R, rank=rank, m_per_rank=M // R,
              seg_order=order, chunk_rows=M // R, n_chunks=1)
    out = _dump(push_ctas=32, push_skip_rounds=1, **kw)
    seen = [(t[0], t[1]) for cta in out for t in cta]
    assert len(seen) == len(set(seen)) and set(seen) == _tiles(M, N, 256)
    rows_per_seg = (M // R) // BM
    for cta in out:                       # source segments are visited in the order of the table
        segs = [order.index(t[0] // rows_per_seg) for t in cta]
        assert segs == sorted(segs)
    first_pos = [cta[0][4] for cta in out if cta]
    workers = len(out) // 2
    early = workers - 16                  # 32 pushing CTAs = 16 pairs sit out the first round
    assert all(p >= early for p in first_pos[:32]) and all(p < early for p in first_pos[32:])
    no_push = _dump(push_ctas=0, **kw)    # without the late join every worker starts in round 0
    assert sorted(cta[0][4] for cta in no_push) == sorted(list(range(len(no_push) // 2)) * 2)


@pytest.mark.parametrize("R,interleave", [(4, 1), (8, 1), (8, 0)])
def test_two_shot_owners(R, interleave):
    M, N, rank = 4096, 8192, 3 % R
    out = _dump(op=OP_AR2, sched=SCHED_STRIDED, M=M, N=N, bn=256, R=R, rank=rank,
                seg_order=rotation_order(rank, R, 1, own_last=True), strided_interleave=interleave)
    tiles = [t for cta in out for t in cta]
    assert set((t[0], t[1]) for t in tiles) == _tiles(M, N, 256)
    tickets = [t[2] for t in tiles]
    assert len(tickets) == len(set(tickets)) and max(tickets) < len(tiles)
    owned = [0] * R
    for t in tiles:
        owned[t[3] % R] += 1
    assert max(owned) - min(owned) <= 2          # CTA tiles (two per pair unit) spread evenly over the owners
    if not interleave:                            # own tiles come last on every worker
        for cta in out:
            own = [t[3] % R == rank for t in cta]
            assert own == sorted(own)


def test_reduce_scatter_walks_own_segment_last():
    R, rank, M, N = 8, 5, 8192, 12288
    order = rotation_order(rank, R, 1, own_last=True)
    out = _dump(op=OP_RS, sched=SCHED_SEGMENT, M=M, N=N, bn=256, R=R, rank=rank, m_per_rank=M // R, seg_order=order)
    rows_per_seg = (M // R) // BM
    for cta in out:
        owners = [t[0] // rows_per_seg for t in cta]
        assert owners[-1] == rank or rank not in owners
        assert [order.index(o) for o in owners] == sorted(order.index(o) for o in owners)
