"""Prompt-cache session: one reusable prompt boundary (KV rows + GDN states) guarded by a small
state machine.

Behaviour of the reference's ``CachedSession`` (``nex_n2_5_pro/sglang_prefill/cache_lifecycle.py:
112-413``): phases ``EMPTY -> FILLING -> READY -> DECODING -> READY``; a new request is served as

* ``HIT``     the retained boundary is exactly the request's prompt,
* ``APPEND``  the retained boundary is a proper prefix of the prompt (only the suffix is prefilled),
* ``PREFILL`` anything else (a shorter prefix can never be reused: the gated-delta-net state
  cannot be rewound),

and reuse additionally requires the same owner key, the same model epoch and a live observation of
the device boundary equal to the one stored when the boundary was last restored.  Every phase
change is made under a lease so that a stale caller cannot commit into a newer request.

The implementation is a transition table over immutable records; the engine-facing part (what a
"boundary" observes) is just three integers read from the control block.
"""

from __future__ import annotations

import hashlib
import threading
from dataclasses import dataclass, replace
from enum import Enum
from typing import Iterable, Optional, Tuple


class CachePhase(str, Enum):
    EMPTY = "empty"
    FILLING = "filling"
    READY = "ready"
    DECODING = "decoding"


class CacheDecision(str, Enum):
    PREFILL = "prefill"
    APPEND = "append"
    HIT = "hit"


class CacheLeaseError(RuntimeError):
    """A lease that is stale, foreign or used in the wrong phase."""


class CacheBusyError(RuntimeError):
    """A request arrived while another one owns the cache."""


@dataclass(frozen=True)
class CacheBoundary:
    """What the device says about the retained prompt boundary."""

    committed_len: int          # control-block committed length
    first_token: int            # pending token at the boundary
    state_tag: int              # cheap checksum of the recurrent state (0 if unused)

    def as_record(self) -> Tuple[int, int, int]:
        return (int(self.committed_len), int(self.first_token), int(self.state_tag))


@dataclass(frozen=True)
class CachePlan:
    generation: int
    decision: CacheDecision
    base_length: int            # tokens already in the cache that will be kept
    target_length: int


@dataclass(frozen=True)
class CacheLease:
    generation: int
    request_id: str
    decision: CacheDecision
    base_length: int
    target_length: int


@dataclass(frozen=True)
class CachedSessionSnapshot:
    phase: CachePhase
    generation: int
    owner: Optional[str]
    model_epoch: Optional[str]
    committed_tokens: Tuple[int, ...]
    token_digest: Optional[str]
    valid_kv_length: int
    boundary: Optional[CacheBoundary]
    last_error: Optional[str]


def token_digest(tokens: Iterable[int]) -> Optional[str]:
    toks = tuple(int(t) for t in tokens)
    if not toks:
        return None
    h = hashlib.blake2b(digest_size=16)
    for t in toks:
        h.update(t.to_bytes(8, "little", signed=True))
    return h.hexdigest()


_EMPTY = CachedSessionSnapshot(CachePhase.EMPTY, 0, None, None, (), None, 0, None, None)


class CachedSession:
    def __init__(self, capacity: int, model_epoch: str):
        if int(capacity) < 1:
            raise ValueError("capacity must be >= 1")
        if not str(model_epoch):
            raise ValueError("model_epoch must not be empty")
        self.capacity, self.model_epoch = int(capacity), str(model_epoch)
        self._s = _EMPTY
        self._lease: Optional[CacheLease] = None
        self._target: Tuple[int, ...] = ()
        self._lock = threading.RLock()

    # ---- read side ----------------------------------------------------------------------------------
    def snapshot(self) -> CachedSessionSnapshot:
        with self._lock:
            return self._s

    def _normalise(self, owner, tokens, model_epoch):
        target = tuple(int(t) for t in tokens)
        if not target:
            raise ValueError("cache request must contain at least one token")
        if len(target) > self.capacity:
            raise ValueError(f"request length {len(target)} exceeds cache capacity {self.capacity}")
        if owner is not None:
            owner = str(owner)
            if not owner:
                raise ValueError("owner must be non-empty or None")
        epoch = self.model_epoch if model_epoch is None else str(model_epoch)
        if not epoch:
            raise ValueError("model_epoch must not be empty")
        return owner, target, epoch

    def _reusable(self, owner, epoch, target, live: Optional[CacheBoundary]) -> bool:
        s = self._s
        n = len(s.committed_tokens)
        return bool(
            owner is not None and s.phase == CachePhase.READY and s.owner == owner and s.model_epoch == epoch and n > 0
            and s.valid_kv_length == n and s.boundary is not None and live == s.boundary and n <= len(target)
            and target[:n] == s.committed_tokens
        )

    def _plan(self, owner, target, epoch, live) -> CachePlan:
        if self._s.phase in (CachePhase.FILLING, CachePhase.DECODING):
            raise CacheBusyError(f"cache is currently {self._s.phase.value}")
        if self._reusable(owner, epoch, target, live):
            base = len(self._s.committed_tokens)
            decision = CacheDecision.HIT if base == len(target) else CacheDecision.APPEND
        else:
            base, decision = 0, CacheDecision.PREFILL
        return CachePlan(self._s.generation + 1, decision, base, len(target))

    def plan_request(self, owner, tokens, *, model_epoch=None, live_boundary: Optional[CacheBoundary] = None) -> CachePlan:
        """The decision the next request would get, without changing phase (used for TP consensus)."""
        owner, target, epoch = self._normalise(owner, tokens, model_epoch)
        with self._lock:
            return self._plan(owner, target, epoch, live_boundary)

    # ---- write side ---------------------------------------------------------------------------------
    def begin_request(self, owner, tokens, request_id: str, *, model_epoch=None, live_boundary=None, force_prefill: bool = False) -> CacheLease:
        owner, target, epoch = self._normalise(owner, tokens, model_epoch)
        with self._lock:
            plan = self._plan(owner, target, epoch, live_boundary)
            if force_prefill and plan.decision != CacheDecision.PREFILL:
                plan = CachePlan(plan.generation, CacheDecision.PREFILL, 0, plan.target_length)
            lease = CacheLease(plan.generation, str(request_id), plan.decision, plan.base_length, plan.target_length)
            if plan.decision == CacheDecision.PREFILL:
                kept: Tuple[int, ...] = ()
                boundary = None
            else:
                kept, boundary = self._s.committed_tokens, self._s.boundary
            self._s = CachedSessionSnapshot(CachePhase.FILLING, plan.generation, owner, epoch, kept, token_digest(kept), len(kept), boundary, None)
            self._lease, self._target = lease, target
            return lease

    def _check(self, lease: CacheLease, phase: CachePhase) -> None:
        if self._lease is None or lease != self._lease or lease.generation != self._s.generation:
            raise CacheLeaseError("stale or foreign cache lease")
        if self._s.phase != phase:
            raise CacheLeaseError(f"cache is {self._s.phase.value}, expected {phase.value}")

    def record_append(self, lease: CacheLease, start: int, end: int) -> None:
        """Tokens ``[start, end)`` of the target are now in the cache (chunked prefill progress)."""
        with self._lock:
            self._check(lease, CachePhase.FILLING)
            if start != self._s.valid_kv_length or not start < end <= len(self._target):
                raise CacheLeaseError(f"append [{start}, {end}) does not continue valid length {self._s.valid_kv_length}")
            toks = self._target[:end]
            self._s = replace(self._s, committed_tokens=toks, token_digest=token_digest(toks), valid_kv_length=end)

    def _validate(self, lease: CacheLease, boundary: CacheBoundary, length: int) -> None:
        if boundary.committed_len != length:
            raise CacheLeaseError(f"boundary length {boundary.committed_len} != expected {length}")

    def validate_fill_boundary(self, lease: CacheLease, boundary: CacheBoundary) -> None:
        with self._lock:
            self._check(lease, CachePhase.FILLING)
            self._validate(lease, boundary, lease.target_length)

    def commit_fill(self, lease: CacheLease, boundary: CacheBoundary) -> CachedSessionSnapshot:
        with self._lock:
            self._check(lease, CachePhase.FILLING)
            self._validate(lease, boundary, lease.target_length)
            if self._s.valid_kv_length != lease.target_length:
                raise CacheLeaseError("fill committed before every token was appended")
            self._s = replace(self._s, phase=CachePhase.READY, boundary=boundary)
            return self._s

    def abort_fill(self, lease: CacheLease, reason: str) -> CachedSessionSnapshot:
        with self._lock:
            self._check(lease, CachePhase.FILLING)
            return self._clear(reason)

    def begin_decode(self, lease: CacheLease) -> CachedSessionSnapshot:
        with self._lock:
            self._check(lease, CachePhase.READY)
            self._s = replace(self._s, phase=CachePhase.DECODING)
            return self._s

    def validate_decode_boundary(self, lease: CacheLease, boundary: CacheBoundary) -> None:
        with self._lock:
            self._check(lease, CachePhase.DECODING)
            if boundary != self._s.boundary:
                raise CacheLeaseError("restored boundary differs from the committed one")

    def finish_decode(self, lease: CacheLease, boundary: CacheBoundary) -> CachedSessionSnapshot:
        """Decode is over and the prompt boundary has been restored on the device."""
        with self._lock:
            self._check(lease, CachePhase.DECODING)
            if boundary != self._s.boundary:
                return self._clear("boundary not restored after decode")
            self._s = replace(self._s, phase=CachePhase.READY)
            self._lease = None
            return self._s

    def abort_decode(self, lease: CacheLease, reason: str) -> CachedSessionSnapshot:
        with self._lock:
            self._check(lease, CachePhase.DECODING)
            return self._clear(reason)

    def invalidate(self, reason: str = "invalidated", *, force: bool = False) -> CachedSessionSnapshot:
        with self._lock:
            if self._s.phase in (CachePhase.FILLING, CachePhase.DECODING) and not force:
                raise CacheBusyError(f"cannot invalidate a cache that is {self._s.phase.value}")
            return self._clear(reason)

    def _clear(self, reason: Optional[str]) -> CachedSessionSnapshot:
        self._s = replace(_EMPTY, generation=self._s.generation, last_error=reason)
        self._lease, self._target = None, ()
        return self._s
