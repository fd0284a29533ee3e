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
    out = _dump(M=8192, N=6144, bn=256, allow_wide=0)
    for even, odd in zip(out[0::2], out[1::2]):
        assert [(t[0] + 1, t[1]) for t in even] == [(t[0], t[1]) for t in odd]
        assert all(t[0] % 2 == 0 for t in even)


def test_wide_pairs_take_four_adjacent_row_blocks():
    """512 x 256 tiles per CTA pair: each CTA owns two consecutive 128-row blocks, the second
    CTA of the pair the two that follow."""
    out = _dump(M=8192, N=6144, bn=256)
    for even, odd in zip(out[0::2], out[1::2]):
        assert len(even) % 2 == 0 and len(even) == len(odd)
        for a, b in zip(even[0::2], even[1::2]):
            assert a[0] % 4 == 0 and (b[0], b[1]) == (a[0] + 1, a[1])
        assert [(t[0] + 2, t[1]) for t in even] == [(t[0], t[1]) for t in odd]


@pytest.mark.parametrize("M,N,K,bn,pair", [(8192, 6144, 12288, 256, 1), (128, 8192, 3584, 256, 1),
                                           (128, 8192, 28672, 128, 1), (4096, 8192, 3584, 256, 1),
                                           (1024, 8192, 3584, 128, 1), (8192, 6144, 12288, 256, 0)])
def test_remainder_round_is_cut_along_k(M, N, K, bn, pair):
    """The tiles of the last, partial round are cut into K ranges on consecutive workers: the
    ranges of a tile partition its k-blocks, slice 0 is the worker that also appears in the tile
    schedule, and no worker takes more than one slice."""
    from tridist_b200.parallel.runtime import native
    d = dict(op=OP_PLAIN, sched=SCHED_NATURAL, bn=bn, R=1, rank=0, M=M, N=N, K=K, allow_pair=pair)
    cuts = native().splitk_dump(d, 148)
    out = _dump(M=M, N=N, K=K, bn=bn, allow_pair=pair)
    seen = [(t[0], t[1]) for cta in out for t in cta if t[0] * BM < M]
    assert len(seen) == len(set(seen)) and set(seen) == _tiles(M, N, bn)
    assert cuts, "these shapes leave a partial round"
    k_blocks = (K + 63) // 64
    by_pos = {}
    for pos, cta0, sl, n, kb0, kb1 in cuts:
        by_pos.setdefault(pos, []).append((sl, n, kb0, kb1, cta0))
    workers = [c[1] for c in cuts]
    assert len(workers) == len(set(workers))
    finisher_pos = {t[4]: c for c, cta in enumerate(out) for t in cta}
    for pos, parts in by_pos.items():
        parts.sort()
        n = parts[0][1]
        assert [q[0] for q in parts] == list(range(n)) and 2 <= n <= 8
        assert parts[0][2] == 0 and parts[-1][3] == k_blocks
        assert all(a[3] == b[2] for a, b in zip(parts, parts[1:]))
        assert all(q[3] - q[2] >= 8 for q in parts)
        step = parts[1][4] - parts[0][4]
        assert [q[4] for q in parts] == [parts[0][4] + i * step for i in range(n)]
        assert finisher_pos[pos] // step * step == parts[0][4]


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
    assert max(owned) - min(owned) <= 4          # 128-row blocks (four per pair unit) spread evenly over the owners
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


@pytest.mark.parametrize("R", [4, 8])
def test_reduce_scatter_through_the_switch_walks_owners_in_lockstep(R):
    """Same order on every rank: position i is tile i // R of owner i % R, so the R partials of a tile
    are produced at about the same time everywhere and the owner can sum them right away."""
    M, N = 8192, 12288
    dumps = []
    for rank in (0, R - 1):
        out = _dump(op=OP_RS, sched=SCHED_SEGMENT, M=M, N=N, bn=256, R=R, rank=rank, m_per_rank=M // R,
                    seg_order=list(range(R)), seg_interleave=1, nvls=1, slot_stride=0)
        dumps.append(out)
        seen = [(t[0], t[1]) for cta in out for t in cta]
        assert len(seen) == len(set(seen)) and set(seen) == _tiles(M, N, 256)
    assert dumps[0] == dumps[1]
    rows_per_seg = (M // R) // BM
    by_pos = sorted({(t[4], t[0] // rows_per_seg) for cta in dumps[0] for t in cta})
    owners = [o for _, o in by_pos]
    assert owners[:2 * R] == list(range(R)) * 2


def test_own_first_band_major_walk():
    """The walk of the multicast all-gather: the rank's own segment whole, then row unit b of every
    other source (in the order's sequence) before row unit b + 1 of any. Every tile exactly once."""
    R, rank, M, N = 8, 2, 8192, 6144
    order = rotation_order(rank, R, 1, own_last=False)
    out = _dump(op=OP_AG, sched=SCHED_SEGMENT, R=R, rank=rank, M=M, N=N, K=12288, m_per_rank=M // R,
                seg_order=order, seg_bands=-1, seg_own_first=1, allow_splitk=0)
    seen = [(t[0], t[1]) for cta in out for t in cta]
    assert len(seen) == len(set(seen)) and set(seen) == _tiles(M, N, 256)
    # positions are dealt round-robin: item i of worker w is position i * workers + w; a worker is a
    # CTA pair whose two CTAs hold two row blocks each (512-row units)
    workers = len(out) // 2
    by_pos = {}
    for w in range(workers):
        for i, t in enumerate(out[2 * w][0::2]):
            by_pos[i * workers + w] = t[0] // 4          # row unit of the position
    units = [by_pos[k] for k in sorted(by_pos)]
    seg_units = (M // R) // 512
    n_tiles = N // 256
    src_of = [u // seg_units for u in units]
    band_of = [u % seg_units for u in units]
    own = seg_units * n_tiles
    assert set(src_of[:own]) == {rank}
    bands = band_of[own:]
    assert bands == sorted(bands), "band b of every other source before band b + 1 of any"
    assert rank not in src_of[own:]
    # inside a band the area of all other sources is walked in groups, column by column: the
    # tiles of one round of 74 workers share a handful of B column blocks
    first_round = [t for w in range(workers) for t in out[2 * w][0:2]][0::2]
    later = [by_pos[k] for k in sorted(by_pos) if own <= k < own + workers]
    assert len(set(later)) >= 3, "several sources side by side"
