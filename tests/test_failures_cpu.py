"""Failure detection without any GPU fault: every failure is made on the host.

* a rank that leaves between steps announces it on the liveness board; its peers learn of it
  before their next launch and do not enter the collective
* a rank that vanishes without a word ends the peers' next collective with an error after a
  short process-group timeout instead of a hang
* an oversubscribed MoE receive buffer is reported as an error
* a silent peer is found by the heartbeat watchdog
"""
import os
import tempfile
import time

import pytest
import torch

from tridist_b200.utils.testing import moe_inputs, randn_seeded, spawn


def _leave_announced(rank, R, outdir):
    from tridist_b200.ops import ag_gemm_intra_node, create_ag_gemm_intra_node_context
    from tridist_b200.parallel.liveness import LivenessBoard, PeerLeft
    from tridist_b200.parallel.runtime import CpuWorld
    w = CpuWorld(rank, R)
    board = LivenessBoard(rank, R)
    ctx = create_ag_gemm_intra_node_context(128 * R, 64, torch.float32, torch.float32, rank, R, M_PER_CHUNK=128, world=w)
    a, b = randn_seeded((128, 64), rank), randn_seeded((32, 64), 9)
    board.check_peers()
    ag_gemm_intra_node(a, b, False, ctx)              # step 1: everybody is there
    torch.distributed.barrier()
    if rank == 1:
        board.announce_leave("test: leaving between steps")
    else:
        deadline = time.time() + 20
        outcome = "no-signal"
        while time.time() < deadline:
            try:
                board.check_peers()
            except PeerLeft as e:
                outcome = "peer-left:" + str(e)
                break
            time.sleep(0.05)
        with open(os.path.join(outdir, "rank0.txt"), "w") as fh:
            fh.write(outcome)
    # nobody enters step 2; both ranks still meet at the final barrier of the launcher


def _vanish(rank, R, outdir):
    from tridist_b200.ops import ag_gemm_intra_node, create_ag_gemm_intra_node_context
    from tridist_b200.parallel.runtime import CpuWorld
    w = CpuWorld(rank, R)
    ctx = create_ag_gemm_intra_node_context(128 * R, 64, torch.float32, torch.float32, rank, R, M_PER_CHUNK=128, world=w)
    a, b = randn_seeded((128, 64), rank), randn_seeded((32, 64), 9)
    ag_gemm_intra_node(a, b, False, ctx)
    torch.distributed.barrier()
    if rank == 1:
        os._exit(0)                                   # gone without a word, nothing in flight
    t0 = time.time()
    try:
        ag_gemm_intra_node(a, b, False, ctx)
        outcome = "completed"
    except Exception as e:  # noqa: BLE001
        outcome = f"error after {time.time() - t0:.1f}s: {type(e).__name__}"
    with open(os.path.join(outdir, "rank0.txt"), "w") as fh:
        fh.write(outcome)
    os._exit(0)


def test_peer_leave_is_seen_before_launch():
    with tempfile.TemporaryDirectory() as d:
        spawn(_leave_announced, 2, args=(d,))
        assert open(os.path.join(d, "rank0.txt")).read().startswith("peer-left:rank(s) [1]")


def test_vanished_peer_ends_collective_with_error():
    with tempfile.TemporaryDirectory() as d:
        try:
            spawn(_vanish, 2, args=(d,), timeout=120, pg_timeout_s=8)
        except RuntimeError:
            pass                                      # the launcher may report the hard exits
        out = open(os.path.join(d, "rank0.txt")).read()
        assert out.startswith("error after"), out
        assert float(out.split()[2][:-2]) < 60


def test_moe_receive_overflow_is_reported():
    from tridist_b200.ops import create_moe_a2a_intra_node_context, moe_dispatch_intra_node_op
    from tridist_b200.parallel.runtime import CpuWorld
    w = CpuWorld(0, 1)
    ctx = create_moe_a2a_intra_node_context(4, 16, torch.float32, 8, 2, 0, 1, world=w, max_recv_rows=5)
    tokens, idx, _ = moe_inputs(0, 8, 16, 4, 2, 0, torch.float32)
    with pytest.raises(RuntimeError, match="oversubscribed"):
        moe_dispatch_intra_node_op(tokens, idx, ctx)


def test_heartbeat_finds_silent_peer():
    from torch.distributed import HashStore
    from tridist_b200.parallel.liveness import LivenessBoard
    store = HashStore()
    b0, b1 = LivenessBoard(0, 2, store), LivenessBoard(1, 2, store)
    b1.beat()
    assert b0.stale_peers(0.2) == []
    time.sleep(0.3)
    b1.beat()                                         # still alive
    assert b0.stale_peers(0.2) == []
    time.sleep(0.3)
    assert b0.stale_peers(0.2) == [1]                 # no beat since the last look


def _multicast_one_rank_cannot(rank, R, outdir):
    """ProcessWorld.alloc_multicast with a stand-in allocator that fails on rank 1: every rank must
    come back with None (and the reason), none may enter the allocator's rendezvous."""
    from tridist_b200.parallel import runtime

    class FakeSymm:
        rendezvous_calls = 0

        @staticmethod
        def empty(n, dtype=None, device=None):
            if rank == 1:
                raise RuntimeError("no multicast on this rank")
            return torch.empty(n, dtype=torch.uint8)

        @staticmethod
        def rendezvous(t, group):
            FakeSymm.rendezvous_calls += 1
            raise AssertionError("rendezvous entered although a rank could not allocate")

    runtime._symm_mem_module = lambda: FakeSymm
    os.environ["TRIDIST_MC_ALLOC"] = "torch"                    # the path through torch's allocator
    w = runtime.ProcessWorld.__new__(runtime.ProcessWorld)      # host logic only: no device, no heap
    runtime._WorldBase.__init__(w)
    w.rank, w.num_ranks, w.group, w.device = rank, R, None, 0
    got = runtime.ProcessWorld.alloc_multicast(w, 4096)
    with open(os.path.join(outdir, f"rank{rank}.txt"), "w") as fh:
        fh.write(f"{got is None}|{FakeSymm.rendezvous_calls}|{getattr(w, 'multicast_unavailable', '')}")


def test_multicast_allocation_fails_on_all_ranks_together():
    with tempfile.TemporaryDirectory() as d:
        spawn(_multicast_one_rank_cannot, 2, args=(d,), timeout=60)
        for r in range(2):
            none, calls, why = open(os.path.join(d, f"rank{r}.txt")).read().split("|", 2)
            assert none == "True" and calls == "0"
            assert "rank 1" in why and "no multicast on this rank" in why
