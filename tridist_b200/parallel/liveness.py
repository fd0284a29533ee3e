"""Host-side liveness board: ranks announce that they leave, peers check before launching.

The fused kernels wait for their peers inside the kernel (bounded, reported through
the status plane). A rank that stops between steps would therefore cost every other
rank one full wait limit per launch. The board avoids that: a rank that leaves on
purpose (or catches an exception) writes a key to the job's key-value store, and
``check_peers`` — called on the host before a launch — raises ``PeerLeft`` as soon as
any peer did so. It also carries a heartbeat counter per rank for watchdogs that want
to detect silent peers (``stale_peers``). The reference has no rank-failure handling;
its tests rely on ``timeout N mpirun`` and a stream watchdog
(tests/test_gemm_ar_rd.py:94-104, tests/dbg_rs_big.py:66-182).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch.distributed as dist


class PeerLeft(RuntimeError):
    """A peer announced that it left the job (or was marked dead by a watchdog)."""


class LivenessBoard:
    def __init__(self, rank: int, num_ranks: int, store=None, prefix: str = "tridist/live"):
        if store is None:
            if not dist.is_initialized():
                raise RuntimeError("LivenessBoard needs an initialised process group or an explicit store")
            store = dist.distributed_c10d._get_default_store()
        self.store, self.rank, self.num_ranks, self.prefix = store, rank, num_ranks, prefix
        self._beats = 0
        self._last_seen: Dict[int, tuple] = {}
        self.store.add(f"{prefix}/left_count", 0)

    def _key(self, what: str, r: int) -> str:
        return f"{self.prefix}/{what}/{r}"

    # -- leaving ---------------------------------------------------------------
    def announce_leave(self, reason: str = "") -> None:
        """Call between steps, with none of this rank's kernels or collectives in flight."""
        self.store.set(self._key("left", self.rank), reason or "left")
        self.store.add(f"{self.prefix}/left_count", 1)

    def left_peers(self) -> List[int]:
        if int(self.store.add(f"{self.prefix}/left_count", 0)) == 0:
            return []
        out = []
        for r in range(self.num_ranks):
            if r != self.rank and self.store.check([self._key("left", r)]):
                out.append(r)
        return out

    def check_peers(self) -> None:
        gone = self.left_peers()
        if gone:
            raise PeerLeft(f"rank(s) {gone} left the job; not launching")

    # -- heartbeat ---------------------------------------------------------------
    def beat(self) -> None:
        self._beats += 1
        self.store.set(self._key("beat", self.rank), str(self._beats))

    def stale_peers(self, max_age_s: float) -> List[int]:
        """Peers whose heartbeat value has not changed for more than ``max_age_s`` seconds
        (as seen by this rank's successive calls)."""
        now = time.monotonic()
        stale = []
        for r in range(self.num_ranks):
            if r == self.rank:
                continue
            key = self._key("beat", r)
            val: Optional[bytes] = self.store.get(key) if self.store.check([key]) else None
            seen = self._last_seen.get(r)
            if seen is None or seen[0] != val:
                self._last_seen[r] = (val, now)
            elif now - seen[1] > max_age_s:
                stale.append(r)
        return stale
