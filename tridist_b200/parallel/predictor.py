"""Host-side arrival-order predictor for skew-aware tile scheduling.

Behavioural contract of the reference's ``StickyOrderPredictor``
(triton_dist/kernels/dcu/i1_predictor.py:35-138), re-implemented:

* last-vote family: the straggler of the next round is predicted to be the one
  inferred in the last round;
* an online stickiness estimate over a sliding window (share of consecutive
  observations that agree) gates the prediction: below the threshold the table
  degrades to the no-prediction rotation (never worse than no table);
* cold start (fewer than two observations, or no observation in the last round)
  also yields the rotation;
* when the predicted straggler is this rank itself the rotation is kept (its own
  consumer sees no skew);
* otherwise the order is: own rank first, predicted straggler last, the other
  peers in natural order, and ``mode`` = 1 (source-major wave order).

``table()`` returns a dict ``{seq, degraded, mode, k_eff, order, order_packed, budget,
s_hat, cold, stickiness}``; ``order_packed`` packs the order 4 bits per slot (R <= 16).
The order feeds the fused kernel's device order table (``ops/ag_tr_pred.py``).
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Dict, List, Optional


class StickyOrderPredictor:
    def __init__(self, rank: int, num_ranks: int, window: int = 8, stickiness_threshold: float = 0.6):
        if num_ranks > 16:
            raise ValueError("order packing uses 4 bits per slot: num_ranks must be <= 16")
        self.rank = rank
        self.num_ranks = num_ranks
        self.window = window
        self.stickiness_threshold = stickiness_threshold
        self._obs: Deque[Optional[int]] = deque(maxlen=window)
        self.seq = 0
        self.n_tables = 0
        self.n_degraded = 0
        self.last: Optional[Dict] = None

    # -- input ---------------------------------------------------------------
    def observe(self, straggler_inferred: Optional[int]) -> None:
        """One call per round, before ``table()``: the rank that arrived last as seen from
        here, or None when nothing could be inferred."""
        self._obs.append(straggler_inferred)

    @property
    def history(self) -> List[Optional[int]]:
        return list(self._obs)

    # -- derived quantities ----------------------------------------------------
    def rotation(self) -> List[int]:
        """No-prediction order: own rank first, then ranks in increasing cyclic order."""
        return [(self.rank + i) % self.num_ranks for i in range(self.num_ranks)]

    def stickiness(self) -> Optional[float]:
        seen = [s for s in self._obs if s is not None]
        if len(seen) < 2:
            return None
        agree = sum(1 for prev, cur in zip(seen, seen[1:]) if prev == cur)
        return agree / (len(seen) - 1)

    def predict(self):
        """-> (predicted straggler or None, degraded, cold)."""
        if len(self._obs) < 2 or self._obs[-1] is None:
            return None, False, True
        st = self.stickiness()
        return self._obs[-1], (st is not None and st < self.stickiness_threshold), False

    # -- output ------------------------------------------------------------------
    def table(self, k_eff: int, budget_default: int = 128) -> Dict:
        s_hat, degraded, cold = self.predict()
        if cold or degraded or s_hat is None or s_hat == self.rank:
            mode, order = 0, self.rotation()
        else:
            middle = [r for r in range(self.num_ranks) if r != self.rank and r != s_hat]
            mode, order = 1, [self.rank] + middle + [s_hat]
        self.seq += 1
        self.n_tables += 1
        self.n_degraded += 1 if degraded else 0
        packed = 0
        for slot, r in enumerate(order):
            packed |= int(r) << (4 * slot)
        self.last = dict(seq=self.seq, degraded=int(degraded), mode=mode, k_eff=int(k_eff), order=order,
                         order_packed=packed, budget=budget_default, s_hat=s_hat, cold=cold,
                         stickiness=self.stickiness())
        return self.last

    def stats(self) -> Dict:
        return dict(rank=self.rank, n_tables=self.n_tables, n_degraded=self.n_degraded,
                    degrade_rate=(self.n_degraded / self.n_tables) if self.n_tables else 0.0,
                    window=self.window, stickiness_threshold=self.stickiness_threshold,
                    last_stickiness=self.stickiness())


def infer_straggler(arrival_ns: List[int], rank: int) -> Optional[int]:
    """The source whose shard was first seen latest (None if no remote stamp was recorded).

    ``arrival_ns[s]`` is the ``globaltimer`` value at which this rank's kernel first found
    source s's ticket raised; unset entries hold the int64 maximum.
    """
    unset = (1 << 63) - 1
    best, best_t = None, -1
    for s, t in enumerate(arrival_ns):
        if s == rank or t >= unset or t <= 0:
            continue
        if t > best_t:
            best, best_t = s, t
    return best


__all__ = ["StickyOrderPredictor", "infer_straggler"]
