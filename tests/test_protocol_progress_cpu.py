"""Progress of the cross-rank tile protocols, simulated on the replayed schedules of ALL ranks.

An epilogue handles its CTA's tiles strictly in order: it publishes a tile's partial when it gets to
the tile, and where this rank keeps rows of the tile (reduce-scatter) or all of it (one-shot
all-reduce) it then waits for every other rank's partial of that tile before it moves on. If two
ranks could each sit on a tile whose missing partial is behind the other's wait, the kernels would
run into their time limit. The simulation advances every CTA of every rank as far as the rule
allows and demands that all of them finish."""
import pytest

from tridist_b200.ops._gemm_common import (OP_AR1, OP_RS, SCHED_NATURAL, SCHED_SEGMENT, rotation_order)

BM = 128


def _schedules(R, make_desc):
    from tridist_b200.parallel.runtime import native
    C = native()
    out = []
    for r in range(R):
        ctas = C.schedule_dump(make_desc(r), 148)
        out.append([[(t[0], t[1]) for t in cta] for cta in ctas])
    return out


def _run(R, sched, waits_on_tile):
    """sched[r][cta] = tiles in order; waits_on_tile(r, tile) -> True if rank r's epilogue waits there."""
    where = [{t: (c, i) for c, cta in enumerate(sched[r]) for i, t in enumerate(cta)} for r in range(R)]
    ptr = [[0] * len(sched[r]) for r in range(R)]
    progress = True
    while progress:
        progress = False
        for r in range(R):
            for c, cta in enumerate(sched[r]):
                while ptr[r][c] < len(cta):
                    t = cta[ptr[r][c]]
                    if waits_on_tile(r, t):
                        arrived = all(t in where[s] and ptr[s][where[s][t][0]] >= where[s][t][1]
                                      for s in range(R) if s != r)
                        if not arrived:
                            break
                    ptr[r][c] += 1
                    progress = True
    stuck = [(r, c, cta[ptr[r][c]]) for r in range(R) for c, cta in enumerate(sched[r]) if ptr[r][c] < len(cta)]
    return stuck


@pytest.mark.parametrize("R,M,N,bn,pair", [(2, 1024, 768, 256, 1), (8, 8192, 12288, 256, 1), (8, 8192, 12288, 256, 0),
                                          (4, 4096, 1024, 128, 1), (8, 512, 2048, 256, 1), (8, 1536, 1024, 256, 1),
                                          (4, 768, 512, 128, 1)])
def test_reduce_scatter_never_blocks(R, M, N, bn, pair):
    m_pr = M // R

    def desc(r):
        return dict(op=OP_RS, sched=SCHED_SEGMENT if m_pr % BM == 0 else SCHED_NATURAL, bn=bn, R=R, rank=r, M=M, N=N,
                    K=1024, m_per_rank=m_pr, slot_stride=m_pr * N, allow_pair=pair,
                    seg_order=rotation_order(r, R, 1, own_last=True))

    def waits(r, tile):
        row0 = tile[0] * BM
        if row0 >= M:
            return False
        o_lo, o_hi = row0 // m_pr, min((min(row0 + BM, M) - 1) // m_pr, R - 1)
        return o_lo <= r <= o_hi                        # this rank keeps rows of the tile

    assert _run(R, _schedules(R, desc), waits) == []


@pytest.mark.parametrize("R,M,N,bn", [(2, 128, 8192, 128), (8, 1024, 8192, 256), (4, 384, 1024, 256)])
def test_one_shot_all_reduce_never_blocks(R, M, N, bn):
    def desc(r):
        return dict(op=OP_AR1, sched=SCHED_NATURAL, bn=bn, R=R, rank=r, M=M, N=N, K=1024, slot_stride=M * N)

    assert _run(R, _schedules(R, desc), lambda r, tile: tile[0] * BM < M) == []


def test_the_simulation_sees_a_cyclic_wait():
    # two ranks, one CTA each, opposite orders, both waiting on their first tile: stuck by construction
    sched = [[[(0, 0), (1, 0)]], [[(1, 0), (0, 0)]]]
    stuck = _run(2, sched, lambda r, tile: True)
    assert len(stuck) == 2
