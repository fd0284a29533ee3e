"""Progress and slot-safety of the recursive-doubling panel exchange, simulated on the host.

The exchange kernel (csrc/ops/rd_exchange.cu) runs, per rank, panel and slice, the steps

    wait ack[slot, phase] >= prev_ticket      the partner consumed the slot's previous occupant
    push the slice into the partner's staging slot, release arrival[slot, phase] = ticket there
    wait arrival[slot, phase] >= ticket       the partner's slice is in my slot
    add it in place, release ack[slot, phase] = ticket at the partner

for phase = 0 .. log2(R) - 1, with the tickets and the slot bookkeeping of
``tridist_b200/ops/gemm_ar_rd.py`` (reference rules: gemm_ar_rd.py:420-470 of the reference project).
Here R ranks run those steps under random interleavings (a rank's panels stay in order, as its
side stream keeps them) and the test demands that every rank finishes every call, that no
staging region is overwritten before its previous occupant was consumed, and that all ranks end
with the full sum. Several calls with different panel counts share one context, so the fixed
ticket stride and the slot history carried from call to call are exercised too.
"""
import random

import pytest

from tridist_b200.ops.gemm_ar_rd import RdState, partners_of


class _Ctx:                                   # what _advance() needs of a context
    def __init__(self, num_chunks, slots, phases):
        self.rd = RdState(chunk_rows=128, num_chunks=num_chunks, stage_slots=slots, phases=phases, slot_bytes=0,
                          comm_ctas=1, transport="rd", round_stride=num_chunks + 1,
                          last_ticket_per_slot=[0] * slots)


def _tasks(ctx, n_tasks):
    """(slot, ticket, prev_ticket) per panel of one call, as gemm_ar_rd_op derives them."""
    from tridist_b200.ops.gemm_ar_rd import _advance
    base = _advance(ctx, n_tasks)
    out = []
    for i in range(n_tasks):
        slot = i % ctx.rd.stage_slots
        ticket = base + i + 1
        prev, ctx.rd.last_ticket_per_slot[slot] = ctx.rd.last_ticket_per_slot[slot], ticket
        out.append((slot, ticket, prev))
    return out


@pytest.mark.parametrize("R,slots,calls", [(2, 1, (3, 1, 2)), (4, 2, (3, 4, 1)), (8, 2, (5, 2)), (8, 4, (4, 4))])
def test_exchange_makes_progress_and_never_overwrites_unconsumed_data(R, slots, calls):
    phases = R.bit_length() - 1
    num_chunks = max(calls)
    ctxs = [_Ctx(num_chunks, slots, phases) for _ in range(R)]
    arrival = [dict() for _ in range(R)]        # (slot, phase) -> ticket, in the OWNER's memory
    ack = [dict() for _ in range(R)]
    staged = [dict() for _ in range(R)]         # (slot, phase) -> (ticket, value, consumed?)
    rng = random.Random(1234 + R * 10 + slots)
    for call, n_tasks in enumerate(calls):
        plans = [_tasks(ctxs[r], n_tasks) for r in range(R)]
        assert all(p == plans[0] for p in plans), "all ranks derive the same slots and tickets"
        value = [[float((r + 1) * (10 ** 0) + 100 * i + 1000 * call) for i in range(n_tasks)] for r in range(R)]
        expect = [sum(value[r][i] for r in range(R)) for i in range(n_tasks)]
        # program counter per rank: (panel, phase, step) with step in 0..3
        pc = [[0, 0, 0] for _ in range(R)]
        done = [n_tasks == 0] * R
        idle = 0
        while not all(done):
            r = rng.randrange(R)
            if done[r]:
                continue
            i, ph, step = pc[r]
            slot, ticket, prev = plans[r][i]
            q = partners_of(r, R)[ph]
            moved = True
            if step == 0:                       # the partner must have freed my previous push into its slot
                moved = ack[r].get((slot, ph), 0) >= prev
            elif step == 1:                     # push + arrival ticket at the partner
                old = staged[q].get((slot, ph))
                assert old is None or old[2], f"rank {r} overwrites unconsumed data of rank {q} (slot {slot}, phase {ph})"
                staged[q][(slot, ph)] = (ticket, value[r][i], False)
                arrival[q][(slot, ph)] = ticket
            elif step == 2:                     # the partner's slice
                moved = arrival[r].get((slot, ph), 0) >= ticket
            else:                               # accumulate, then hand the region back
                t, v, _ = staged[r][(slot, ph)]
                assert t == ticket, "the staged slice belongs to this panel"
                value[r][i] += v
                staged[r][(slot, ph)] = (t, v, True)
                ack[q][(slot, ph)] = ticket
            if not moved:
                idle += 1
                assert idle < 200000, f"no progress: rank {r} stuck at panel {i} phase {ph} step {step}"
                continue
            idle = 0
            step += 1
            if step == 4:
                step, ph = 0, ph + 1
                if ph == phases:
                    ph, i = 0, i + 1
            pc[r] = [i, ph, step]
            done[r] = i == n_tasks
        for r in range(R):
            assert value[r] == expect, f"call {call}: rank {r} holds {value[r]}, expected {expect}"


def test_partner_sequences_pair_up():
    """In every phase the partner relation is an involution that crosses the phase's bit."""
    for R in (2, 4, 8):
        for ph in range(R.bit_length() - 1):
            for r in range(R):
                q = partners_of(r, R)[ph]
                assert q != r and partners_of(q, R)[ph] == r and (q ^ r) == 1 << ph
