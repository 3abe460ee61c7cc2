"""Prompt-cache state machine and tensor-parallel consensus rules (host only)."""

import pytest

from nexrt_b200.serve.cache_consensus import (CacheConsensusError, FatalTPInvariantError, RecoverableRequestError, boundary_record,
                                              failure_record, request_fingerprint, request_record, resolve_boundary, resolve_failure,
                                              resolve_request, resolve_request_outcome, resolve_retain, retain_record)
from nexrt_b200.serve.cache_lifecycle import (CacheBoundary, CacheBusyError, CacheDecision, CachedSession, CacheLeaseError, CachePhase,
                                              CachePlan, token_digest)


def _fill(cache, owner, toks, first=7):
    lease = cache.begin_request(owner, toks, "r", live_boundary=_live(cache))
    if lease.base_length < len(toks):
        cache.record_append(lease, lease.base_length, len(toks))
    b = CacheBoundary(len(toks), first, 0)
    cache.commit_fill(lease, b)
    return lease, b


def _live(cache):
    return cache.snapshot().boundary


def _serve(cache, owner, toks, first=7):
    lease, b = _fill(cache, owner, toks, first)
    cache.begin_decode(lease)
    cache.finish_decode(lease, b)
    return lease


def test_prefill_then_hit_then_append():
    c = CachedSession(64, "m1")
    assert c.snapshot().phase == CachePhase.EMPTY
    l1 = _serve(c, "alice", [1, 2, 3])
    assert l1.decision == CacheDecision.PREFILL and c.snapshot().phase == CachePhase.READY
    assert c.snapshot().token_digest == token_digest([1, 2, 3])
    plan = c.plan_request("alice", [1, 2, 3], live_boundary=_live(c))
    assert plan == CachePlan(2, CacheDecision.HIT, 3, 3)
    l2 = _serve(c, "alice", [1, 2, 3])
    assert l2.decision == CacheDecision.HIT
    l3 = _serve(c, "alice", [1, 2, 3, 4, 5])
    assert (l3.decision, l3.base_length, l3.target_length) == (CacheDecision.APPEND, 3, 5)
    assert c.snapshot().committed_tokens == (1, 2, 3, 4, 5)


@pytest.mark.parametrize(
    "owner,toks,epoch,live_ok",
    [("bob", [1, 2, 3], None, True),          # other owner
     (None, [1, 2, 3], None, True),           # anonymous requests never reuse
     ("alice", [1, 2], None, True),           # shorter prompt: the recurrent state cannot be rewound
     ("alice", [1, 9, 3, 4], None, True),     # not a prefix
     ("alice", [1, 2, 3], "m2", True),        # other weights
     ("alice", [1, 2, 3], None, False)],      # the device boundary is not the stored one
)
def test_reuse_conditions(owner, toks, epoch, live_ok):
    c = CachedSession(64, "m1")
    _serve(c, "alice", [1, 2, 3])
    live = _live(c) if live_ok else CacheBoundary(3, 8, 0)
    assert c.plan_request(owner, toks, model_epoch=epoch, live_boundary=live).decision == CacheDecision.PREFILL


def test_busy_and_stale_leases():
    c = CachedSession(16, "m")
    lease = c.begin_request("a", [1, 2], "r1")
    with pytest.raises(CacheBusyError):
        c.begin_request("a", [1, 2], "r2")
    with pytest.raises(CacheBusyError):
        c.invalidate("x")
    with pytest.raises(CacheLeaseError):
        c.record_append(lease, 1, 2)                  # does not continue valid length 0
    c.record_append(lease, 0, 1)
    with pytest.raises(CacheLeaseError):
        c.commit_fill(lease, CacheBoundary(2, 5, 0))  # one token still missing
    c.record_append(lease, 1, 2)
    with pytest.raises(CacheLeaseError):
        c.commit_fill(lease, CacheBoundary(3, 5, 0))  # wrong length
    with pytest.raises(CacheLeaseError):
        c.begin_decode(lease)                         # still filling
    c.commit_fill(lease, CacheBoundary(2, 5, 0))
    c.begin_decode(lease)
    c.invalidate("forced", force=True)
    assert c.snapshot().phase == CachePhase.EMPTY and c.snapshot().last_error == "forced"
    with pytest.raises(CacheLeaseError):
        c.finish_decode(lease, CacheBoundary(2, 5, 0))
    # generations keep counting through a clear
    assert c.begin_request("a", [1], "r3").generation == 2


def test_decode_that_does_not_restore_clears_the_cache():
    c = CachedSession(16, "m")
    lease, b = _fill(c, "a", [1, 2, 3])
    c.begin_decode(lease)
    with pytest.raises(CacheLeaseError):
        c.validate_decode_boundary(lease, CacheBoundary(3, 9, 0))
    snap = c.finish_decode(lease, CacheBoundary(4, 7, 0))
    assert snap.phase == CachePhase.EMPTY and "not restored" in snap.last_error


def test_force_prefill_and_abort_fill_and_capacity():
    c = CachedSession(4, "m")
    _serve(c, "a", [1, 2])
    lease = c.begin_request("a", [1, 2, 3], "r", live_boundary=_live(c), force_prefill=True)
    assert lease.decision == CacheDecision.PREFILL and c.snapshot().valid_kv_length == 0
    c.abort_fill(lease, "oops")
    assert c.snapshot().phase == CachePhase.EMPTY
    with pytest.raises(ValueError):
        c.plan_request("a", [1, 2, 3, 4, 5])
    with pytest.raises(ValueError):
        c.plan_request("a", [])
    with pytest.raises(ValueError):
        CachedSession(0, "m")


# ---- consensus ---------------------------------------------------------------------------------------
def _fp(**kw):
    base = dict(owner="a", tokens=[1, 2, 3], model_epoch="m", decode_kind="bs1", max_new_tokens=4, seed=0, temperature=0.6, top_p=0.95)
    base.update(kw)
    return request_fingerprint(**base)


def test_fingerprint_is_stable_and_sensitive():
    assert _fp() == _fp() and -(1 << 63) <= _fp() < (1 << 63)
    for kw in (dict(owner=None), dict(owner="b"), dict(tokens=[1, 2, 4]), dict(model_epoch="n"), dict(decode_kind="mtp"),
               dict(max_new_tokens=5), dict(seed=1), dict(temperature=0.7), dict(top_p=0.9), dict(top_k=5)):
        assert _fp(**kw) != _fp()
    # length-prefixed fields: moving a character between fields changes the hash
    assert _fp(owner="ab", model_epoch="c") != _fp(owner="a", model_epoch="bc")


def test_request_consensus_rules():
    hit, pre = CachePlan(3, CacheDecision.HIT, 5, 5), CachePlan(3, CacheDecision.PREFILL, 0, 5)
    fp = 11
    r = resolve_request([request_record(True, hit, fp)] * 4)
    assert (r.decision, r.base_length, r.forced_prefill) == (CacheDecision.HIT, 5, False)
    # one rank lost its boundary -> everyone prefills
    r = resolve_request([request_record(True, hit, fp), request_record(False, pre, fp)])
    assert r.decision == CacheDecision.PREFILL and r.invalid_ranks == (1,) and r.forced_prefill
    with pytest.raises(FatalTPInvariantError):      # fingerprints differ
        resolve_request([request_record(True, hit, 1), request_record(True, hit, 2)])
    with pytest.raises(FatalTPInvariantError):      # valid proposals disagree
        resolve_request([request_record(True, hit, fp), request_record(True, pre, fp)])
    with pytest.raises(FatalTPInvariantError):      # fatal anywhere
        resolve_request([request_record(True, hit, fp), request_record(True, hit, fp, fatal=True)])
    with pytest.raises(FatalTPInvariantError):      # a recoverable failure must be unanimous
        resolve_request([request_record(True, hit, fp), request_record(True, hit, fp, recoverable_failure=True)])
    with pytest.raises(RecoverableRequestError):
        resolve_request([request_record(True, hit, fp, recoverable_failure=True)] * 2)
    # a rank without a live boundary turns the request into a collective PREFILL, but it cannot hide a disagreement about
    # the generation, the target length or the request itself, nor a malformed proposal of a rank that claims to be valid
    with pytest.raises(FatalTPInvariantError):
        resolve_request([request_record(True, hit, fp), request_record(False, CachePlan(4, CacheDecision.PREFILL, 0, 5), fp)])
    with pytest.raises(FatalTPInvariantError):
        resolve_request([request_record(True, hit, fp), request_record(False, CachePlan(3, CacheDecision.PREFILL, 0, 6), fp)])
    with pytest.raises(FatalTPInvariantError):
        resolve_request([request_record(True, hit, fp), request_record(False, pre, fp + 1)])
    with pytest.raises(FatalTPInvariantError):
        resolve_request([request_record(True, CachePlan(3, CacheDecision.APPEND, 9, 5), fp), request_record(False, pre, fp)])   # base beyond the target
    with pytest.raises(CacheConsensusError):
        resolve_request([])
    with pytest.raises(CacheConsensusError):
        resolve_request([(1, 2, 3)])


def test_boundary_retain_and_outcome_rules():
    b = CacheBoundary(5, 42, 0)
    assert resolve_boundary([boundary_record(True, 3, 5, b)] * 2, "fill") == (3, 5, 5, 42)
    with pytest.raises(CacheConsensusError):
        resolve_boundary([boundary_record(True, 3, 5, b), boundary_record(False, 3, 5, b)], "fill")
    with pytest.raises(CacheConsensusError):
        resolve_boundary([boundary_record(True, 3, 5, b), boundary_record(True, 3, 5, CacheBoundary(5, 43, 0))], "fill")
    with pytest.raises(CacheConsensusError):
        resolve_boundary([boundary_record(True, 3, 5, None)], "fill")
    assert resolve_retain([retain_record(True, 3, 5)] * 2) == (True, ())
    assert resolve_retain([retain_record(True, 3, 5), retain_record(False, 3, 5)]) == (False, (1,))
    with pytest.raises(FatalTPInvariantError):
        resolve_retain([retain_record(True, 3, 5), retain_record(True, 4, 5)])
    ok, bad = failure_record(None, 3, 2, 3), failure_record(True, 3, 2, 3)
    assert resolve_request_outcome([ok, ok]) == ("success", (3, 2, 3, 0))
    assert resolve_request_outcome([bad, bad])[0] == "reset"
    assert resolve_failure([bad, bad]) == (3, 2, 3, 0)
    with pytest.raises(FatalTPInvariantError):
        resolve_request_outcome([ok, bad])
    with pytest.raises(FatalTPInvariantError):
        resolve_request_outcome([failure_record(False, 3, 2, 3)] * 2)
    with pytest.raises(FatalTPInvariantError):
        resolve_request_outcome([ok, failure_record(None, 4, 2, 3)])


def test_random_operation_sequences_keep_the_cache_consistent():
    """Any order of lifecycle calls with any arguments either works or raises one of the documented errors, and the
    snapshot stays sane: the valid length never leaves [0, capacity] and an empty cache holds nothing."""
    import random

    from nexrt_b200.serve.cache_lifecycle import CacheBusyError, CacheLeaseError

    rng = random.Random(3)
    for _ in range(400):
        c = CachedSession(32, "m")
        leases = []
        for step in range(40):
            op = rng.randrange(10)
            lease = rng.choice(leases) if leases else None
            toks = [rng.randrange(4) for _ in range(rng.randrange(0, 40))]
            owner = rng.choice([None, "a", "b", ""])
            b = CacheBoundary(rng.randrange(0, 34), rng.randrange(-1, 5), 0)
            try:
                if op == 0:
                    c.plan_request(owner, toks, live_boundary=rng.choice([None, b]))
                elif op == 1:
                    leases.append(c.begin_request(owner, toks, f"r{step}", live_boundary=rng.choice([None, b]), force_prefill=rng.random() < 0.2))
                elif lease is None:
                    continue
                elif op == 2:
                    c.record_append(lease, rng.randrange(0, 34), rng.randrange(0, 34))
                elif op == 3:
                    c.commit_fill(lease, b)
                elif op == 4:
                    c.abort_fill(lease, "x")
                elif op == 5:
                    c.begin_decode(lease)
                elif op == 6:
                    c.finish_decode(lease, b)
                elif op == 7:
                    c.abort_decode(lease, "x")
                elif op == 8:
                    c.invalidate("x", force=rng.random() < 0.5)
                else:
                    c.validate_decode_boundary(lease, b)
                    c.validate_fill_boundary(lease, b)
            except (CacheLeaseError, CacheBusyError, ValueError):
                pass
            s = c.snapshot()
            assert 0 <= s.valid_kv_length <= 32 and (s.phase != CachePhase.EMPTY or s.valid_kv_length == 0), s
