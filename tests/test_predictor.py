"""Arrival-order predictor: the behavioural cases of the reference's unit test
(tests/test_i1_pred.py:61-92) plus table packing and straggler inference."""
from tridist_b200.parallel.predictor import StickyOrderPredictor, infer_straggler


def test_cold_start_gives_rotation():
    p = StickyOrderPredictor(rank=0, num_ranks=2, window=4)
    t = p.table(k_eff=2)
    assert t["mode"] == 0 and t["cold"] and t["order"] == [0, 1]
    p.observe(1)                      # one observation is still cold
    assert p.table(k_eff=2)["cold"]


def test_sticky_chain_predicts_last_vote():
    p = StickyOrderPredictor(rank=0, num_ranks=2, window=4)
    for _ in range(4):
        p.observe(1)
    t = p.table(k_eff=2)
    assert t["mode"] == 1 and t["order"] == [0, 1] and t["degraded"] == 0 and t["s_hat"] == 1
    assert t["stickiness"] == 1.0


def test_own_rank_predicted_keeps_rotation():
    q = StickyOrderPredictor(rank=1, num_ranks=2, window=4)
    for _ in range(4):
        q.observe(1)
    t = q.table(k_eff=2)
    assert t["mode"] == 0 and t["s_hat"] == 1 and t["order"] == [1, 0]


def test_decorrelated_chain_degrades():
    r = StickyOrderPredictor(rank=0, num_ranks=2, window=4)
    for s in (1, 0, 1, 0):
        r.observe(s)
    t = r.table(k_eff=2)
    assert t["mode"] == 0 and t["degraded"] == 1 and t["stickiness"] < 0.6
    assert r.stats()["n_degraded"] == 1 and r.stats()["degrade_rate"] == 1.0


def test_order_at_eight_ranks_and_packing():
    p = StickyOrderPredictor(rank=2, num_ranks=8)
    for _ in range(3):
        p.observe(5)
    t = p.table(k_eff=4, budget_default=96)
    assert t["order"] == [2, 0, 1, 3, 4, 6, 7, 5]        # own first, straggler last, others natural
    assert t["order_packed"] == sum(o << (4 * i) for i, o in enumerate(t["order"]))
    assert t["budget"] == 96 and t["seq"] == 1
    assert p.table(k_eff=4)["seq"] == 2                   # monotonic sequence number


def test_window_and_missing_observation():
    p = StickyOrderPredictor(rank=0, num_ranks=4, window=3)
    for s in (1, 1, 2, 2, 2):
        p.observe(s)
    assert p.history == [2, 2, 2] and p.stickiness() == 1.0
    p.observe(None)                                       # observer produced nothing: cold this round
    assert p.table(k_eff=1)["cold"]


def test_infer_straggler_from_stamps():
    unset = (1 << 63) - 1
    assert infer_straggler([unset, 1000, 5000, 3000], rank=0) == 2
    assert infer_straggler([unset, unset, unset], rank=1) is None
    assert infer_straggler([9000, 1000, 100], rank=0) == 1   # own slot is ignored
