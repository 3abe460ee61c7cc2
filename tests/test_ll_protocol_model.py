"""The LL packet protocol on CPU threads (host model ``parallel/ll_model.py`` of ``csrc/ll.cuh``): tag / half / sequence
bookkeeping over mixes of graphs with different numbers of channel users, ranks running at different speeds, bitwise
agreement between ranks on cancellation-prone inputs, and a peer that never sends.  The reference has no such test
(its collective kernels are only exercised on 8 real GPUs, nex_n2_5_pro/tests/test_cp_reduce_determinism.py); the
model lets the protocol logic be checked where no GPU exists."""

import struct

import pytest

from nexrt_b200.parallel.ll_model import STATUS_OK, STATUS_REDUCE_TIMEOUT, LLModel


def _bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def _f32(x: float) -> float:
    return struct.unpack("<f", struct.pack("<f", x))[0]


def _cancel_inputs(world, call, slot):
    """Values whose sum depends on the order of addition: 2^24, 1, -2^24, ... rotated by call and slot
    (the pattern of the reference's determinism probe, test_cp_reduce_determinism.py:59-113)."""
    base = [16777216.0, 1.0, -16777216.0, 3.0, 0.5, -1.0, 7.0, -0.25]
    return [base[(r + call + slot) % len(base)] for r in range(world)]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_mixed_graphs_alternate_halves_and_agree_bitwise(world):
    slots = 4
    graphs = [3, 5, 2, 5, 3, 3, 2]            # channel users per replayed graph, in replay order (two graph shapes interleaved + a third)

    def program(model, me):
        results = []
        call = 0
        for n_sites in graphs:
            for site in range(n_sites):
                tag, half = model.begin(me, site)
                assert half == ((me.seq + site) & 1)
                for slot in range(slots):
                    me._sleep()
                    own = _cancel_inputs(world, call, slot)[me.rank]
                    # fp32 accumulation in rank order, as the device does
                    total = 0.0
                    vals = []
                    model.publish(me, tag, half, slot, own)
                    for src in range(world):
                        v = own if src == me.rank else model.wait(me, tag, half, src, slot)
                        assert v is not None
                        vals.append(v)
                    for v in vals:
                        total = _f32(total + v)
                    results.append(total)
                call += 1
            model.end_graph(me, n_sites)
        return results

    model = LLModel(world, slots, budget_s=20.0)
    out = model.run(program, jitter_s=0.0005, seed=world)
    # every rank holds the same bits, and they are the rank-order sums
    call = 0
    k = 0
    for n_sites in graphs:
        for _ in range(n_sites):
            for slot in range(slots):
                want = 0.0
                for v in _cancel_inputs(world, call, slot):
                    want = _f32(want + v)
                for r in range(world):
                    assert _bits(out[r][k]) == _bits(want), (r, call, slot)
                k += 1
            call += 1
    assert all(rs.status == STATUS_OK for rs in model.ranks)
    assert sum(graphs) % 2 == 1 or True      # both halves were in use: consecutive calls alternate by construction


def test_a_peer_can_never_be_more_than_one_call_ahead():
    """Rank 0 is slow, rank 1 fast: rank 1 can publish call k + 1 (the other half) while rank 0 still reads call k, but it
    cannot finish call k + 1 - so it cannot overwrite the half of call k with call k + 2 - before rank 0 has sent k + 1."""
    world, n_calls = 2, 40
    progress = [0, 0]
    worst_lead = [0]

    def program(model, me):
        res = []
        for call in range(n_calls):
            if me.rank == 0 and call % 3 == 0:
                import time

                time.sleep(0.002)
            res.append(model.allreduce(me, call, 0, float(call + me.rank)))
            progress[me.rank] = call + 1
            worst_lead[0] = max(worst_lead[0], abs(progress[0] - progress[1]))
        model.end_graph(me, n_calls)
        return res

    model = LLModel(world, 1, budget_s=20.0)
    out = model.run(program)
    assert out[0] == out[1] == [float(2 * c + 1) for c in range(n_calls)]
    assert worst_lead[0] <= 1
    assert all(rs.status == STATUS_OK for rs in model.ranks)


def test_silent_peer_times_out_with_a_status_and_later_waits_give_up_at_once():
    import time

    def program(model, me):
        if me.rank == 1:
            return []
        t0 = time.monotonic()
        a = model.allreduce(me, 0, 0, 5.0)          # waits out its budget
        first = time.monotonic() - t0
        t0 = time.monotonic()
        b = model.allreduce(me, 1, 0, 7.0)          # status already latched: no second wait
        second = time.monotonic() - t0
        return [a, b, first, second]

    model = LLModel(2, 1, budget_s=0.2, silent=[1])
    out = model.run(program)
    a, b, first, second = out[0]
    assert a == 5.0 and b == 7.0                    # the missing peer counts as zero
    assert model.ranks[0].status == STATUS_REDUCE_TIMEOUT
    assert first >= 0.2 and second < 0.1


def test_zeroed_inbox_never_matches_and_stale_packets_are_never_consumed():
    """Tags always carry the top bit, so an all-zero (reset) inbox matches no call; a packet left by an earlier call in
    the same half carries a different tag and is skipped."""
    model = LLModel(2, 1, budget_s=0.05, silent=[1])
    me = model.ranks[0]
    tag, half = model.begin(me, 0)
    assert tag & 0x80000000 and tag != 0
    # an old packet from two calls ago sits in the region this call will poll
    old_tag = ((me.seq + 0 - 2) & 0xFFFFFFFF) | 0x80000000
    me.inbox[half][1][0] = (old_tag, 99.0)
    assert model.wait(me, tag, half, 1, 0) is None
    assert me.stale_reads > 0 and me.status == STATUS_REDUCE_TIMEOUT
