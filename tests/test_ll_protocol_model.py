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


# ---- block protocol of the wide prefill's all-reduce (csrc/prefill.cu: planes_allreduce_residual_kernel) --------------
from nexrt_b200.parallel.ll_model import BlockModel  # noqa: E402


def _block_value(call, rank, cta, lane):
    return float(((call * 8 + rank) * 64 + cta) * 16 + lane)


@pytest.mark.parametrize("world,parallel", [(2, False), (4, True), (8, False)])
def test_block_protocol_never_reads_data_of_another_call(world, parallel):
    """Untagged data vectors + one tagged flag per CTA: over a mix of graphs with different site counts, CTAs of a call
    side by side in a random start order (a resident grid) or one after the other in index order (a grid larger than the
    machine, dispatched in order), ranks at different speeds: every CTA reads exactly what its peers wrote for that
    call, and all ranks get the same sums."""
    import random

    ctas, width = 5, 3
    graphs = [2, 3, 1, 3, 2, 2]

    def program(model, me):
        rng = random.Random(me.rank * 7 + 1)
        results, call = [], 0
        for n_sites in graphs:
            for site in range(n_sites):
                me._sleep()
                order = list(range(ctas))
                if parallel:
                    rng.shuffle(order)
                c = call
                sums = model.call(me, site, lambda b: [_block_value(c, me.rank, b, j) for j in range(width)],
                                  lambda src, b: [_block_value(c, src, b, j) for j in range(width)], order=order, parallel=parallel)
                results.append(sums)
                call += 1
            model.end_graph(me, n_sites)
        return results

    model = BlockModel(world, ctas, width, budget_s=20.0)
    out = model.run(program, jitter_s=0.0005, seed=world)
    assert all(r.status == STATUS_OK for r in model.ranks) and model.stale_data == [0] * world
    assert all(o == out[0] for o in out)
    call = 0
    for sums in out[0]:
        for b in range(ctas):
            assert sums[b] == [sum(_block_value(call, r, b, j) for r in range(world)) for j in range(width)]
        call += 1


def test_block_protocol_breaks_without_the_kernel_boundary():
    """The model is sharp enough to show why the boundary matters: if a rank starts the next-but-one call (same half)
    before a peer's CTA has read the data of the current one, that CTA reads the wrong call's values."""
    model = BlockModel(2, 1, 2, budget_s=5.0)
    a, b = model.ranks
    val = lambda call, rank: [_block_value(call, rank, 0, j) for j in range(2)]
    # rank 1 publishes call 0 and - ignoring every wait - call 2 (site 2: the same half) before rank 0 has run call 0
    for site in (0, 2):
        tag, half = model.begin(b, site)
        for j, v in enumerate(val(site, 1)):
            a.inbox[half][1][j] = (0, v)
        if site == 0:
            a.inbox[half][1][2] = (tag, 0.0)
    got = model.cta(a, 0, 0, val(0, 0), expect=lambda src: val(0, src))
    assert model.stale_data[0] == 1 and got != [x + y for x, y in zip(val(0, 0), val(0, 1))]


def test_block_protocol_needs_resident_or_in_order_ctas():
    """CTA b waits for CTA b of every peer.  If the CTAs of a call ran one at a time in DIFFERENT orders on two ranks,
    each rank would sit in a CTA whose partner has not started: the waits run out.  The device never does that (a grid
    is dispatched in index order and the launcher's grids fit the machine); the model shows what the kernel relies on."""
    model = BlockModel(2, 2, 1, budget_s=0.3)

    def program(m, me):
        out = m.call(me, 0, lambda b: [1.0], order=[0, 1] if me.rank == 0 else [1, 0])
        m.end_graph(me, 1)
        return out

    model.run(program)
    # the rank whose wait runs out first moves on and publishes what the other one is waiting for
    assert any(r.status == STATUS_REDUCE_TIMEOUT for r in model.ranks)


def test_block_protocol_silent_peer_times_out_and_counts_as_zero():
    model = BlockModel(2, 2, 2, budget_s=0.2, silent=(1,))

    def program(m, me):
        out = m.call(me, 0, lambda b: [1.0 + me.rank, 2.0])
        m.end_graph(me, 1)
        return out

    out = model.run(program)
    assert model.ranks[0].status == STATUS_REDUCE_TIMEOUT and out[0] == [[1.0, 2.0], [1.0, 2.0]]
    assert model.ranks[1].status == STATUS_OK and out[1] == [[3.0, 4.0], [3.0, 4.0]]
