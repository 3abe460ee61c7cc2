"""Tensor-parallel agreement on every cache-lifecycle transition.

Each rank describes what it would do as a short row of int64 words; the rows of all ranks are
all-gathered (host side, NCCL or gloo) and every rank resolves the SAME table with the pure functions
below, so all ranks take the same branch or all raise.  Rules are those of the reference
(``nex_n2_5_pro/sglang_prefill/cache_consensus.py:65-267``):

* request rows ``[validity, decision, generation, base, target, fingerprint]``: generation, target
  and request fingerprint must be identical everywhere (else fatal); validity -1 anywhere is fatal;
  validity -2 must be unanimous and is a recoverable request failure; validity 0 on any rank means
  "my live boundary no longer matches" and turns the request into a collective PREFILL; otherwise the
  valid proposals must agree exactly.
* boundary rows ``[valid, generation, prefill_len, decode_len, pending]`` must all be valid and equal.
* retain rows ``[retain, generation, target, 0, 0]``: the boundary is kept only if every rank agrees.
* outcome rows ``[outcome, generation, phase, active_generation, kind]``: all 2 -> success, all 1 ->
  collective reset, anything mixed -> fatal.

Nothing here touches a GPU or a process group: the functions take lists of rows, which is what makes
the protocol testable on CPU.
"""

from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence, Tuple

from .cache_lifecycle import CacheBoundary, CacheDecision, CachePlan

_CODES = {CacheDecision.PREFILL: 0, CacheDecision.APPEND: 1, CacheDecision.HIT: 2}
_DECISIONS = {v: k for k, v in _CODES.items()}

VALID, LOCAL_MISMATCH, FATAL, RECOVERABLE = 1, 0, -1, -2
REQUEST_WORDS, BOUNDARY_WORDS = 6, 5


class CacheConsensusError(RuntimeError):
    pass


class FatalTPInvariantError(CacheConsensusError):
    """The ranks disagree about something that must be identical: the group cannot continue."""


class RecoverableRequestError(CacheConsensusError):
    """Every rank agrees that this request failed before touching the cache."""


@dataclass(frozen=True)
class RequestConsensus:
    generation: int
    decision: CacheDecision
    base_length: int
    target_length: int
    invalid_ranks: Tuple[int, ...]

    @property
    def forced_prefill(self) -> bool:
        return bool(self.invalid_ranks)


def request_fingerprint(*, owner: Optional[str], tokens: Iterable[int], model_epoch: str, decode_kind: str, max_new_tokens: int,
                        seed: int, temperature: float, top_p: float, handoff_mode: str = "native", top_k: int = 20) -> int:
    """Stable signed 64-bit identity of a request (every rank must have received the same one)."""
    h = hashlib.blake2b(digest_size=8, person=b"nexrt-b200-tp")

    def put(b: bytes) -> None:
        h.update(struct.pack("<Q", len(b)))
        h.update(b)

    put(b"" if owner is None else b"\x01" + str(owner).encode())
    put(str(model_epoch).encode())
    put(str(decode_kind).encode())
    put(str(handoff_mode).encode())
    put(struct.pack("<qqdd q", int(max_new_tokens), int(seed) & ((1 << 63) - 1), float(temperature), float(top_p), int(top_k)))
    toks = [int(t) for t in tokens]
    put(struct.pack(f"<{len(toks)}q", *toks))
    return struct.unpack("<q", h.digest())[0]


def request_record(valid: bool, plan: CachePlan, fingerprint: int, *, fatal: bool = False, recoverable_failure: bool = False):
    validity = FATAL if fatal else (RECOVERABLE if recoverable_failure else int(bool(valid)))
    return (validity, _CODES[plan.decision], int(plan.generation), int(plan.base_length), int(plan.target_length), int(fingerprint))


def boundary_record(valid: bool, lease_generation: int, target_length: int, boundary: Optional[CacheBoundary]):
    if boundary is None:
        return (int(bool(valid)), int(lease_generation), int(target_length), -1, -1)
    return (int(bool(valid)), int(lease_generation), int(target_length), int(boundary.committed_len), int(boundary.first_token))


def retain_record(retain: bool, generation: int, target_length: int):
    return (int(bool(retain)), int(generation), int(target_length), 0, 0)


def failure_record(recoverable: Optional[bool], generation: int, phase: int, active_generation: int, request_kind: int = 0):
    """outcome word: 2 = finished, 1 = failed but collectively resettable, 0 = fatal here."""
    outcome = 2 if recoverable is None else int(bool(recoverable))
    return (outcome, int(generation), int(phase), int(active_generation), int(request_kind))


def _table(rows: Iterable[Sequence[int]], width: int, first_word: Tuple[int, ...]) -> List[Tuple[int, ...]]:
    table = [tuple(int(v) for v in row) for row in rows]
    if not table or any(len(r) != width for r in table):
        raise CacheConsensusError(f"consensus needs a non-empty table of {width}-word rows")
    if any(r[0] not in first_word for r in table):
        raise CacheConsensusError(f"unknown leading word in consensus table: {table}")
    return table


def _same(table, columns: slice) -> bool:
    return len({r[columns] for r in table}) == 1


def resolve_request(rows: Iterable[Sequence[int]]) -> RequestConsensus:
    t = _table(rows, REQUEST_WORDS, (VALID, LOCAL_MISMATCH, FATAL, RECOVERABLE))
    if not (_same(t, slice(2, 3)) and _same(t, slice(4, 6))):
        raise FatalTPInvariantError(f"generation / target / request identity differ across ranks: {t}")
    if any(r[0] == FATAL for r in t):
        raise FatalTPInvariantError(f"fatal proposal on ranks {[i for i, r in enumerate(t) if r[0] == FATAL]}: {t}")
    failed = [i for i, r in enumerate(t) if r[0] == RECOVERABLE]
    if failed:
        if len(failed) != len(t):
            raise FatalTPInvariantError(f"only ranks {failed} report a request failure: {t}")
        raise RecoverableRequestError(f"all ranks rejected the request: {t}")
    generation, target = t[0][2], t[0][4]
    if generation < 1 or target < 1:
        raise FatalTPInvariantError(f"malformed proposal: {t}")
    valid = [r for r in t if r[0] == VALID]
    if any(r[1] not in _DECISIONS or not 0 <= r[3] <= target for r in valid):
        raise FatalTPInvariantError(f"malformed proposal: {t}")
    proposals = {(r[1], r[3]) for r in valid}
    if len(proposals) > 1:
        raise FatalTPInvariantError(f"valid proposals disagree: {t}")
    invalid = tuple(i for i, r in enumerate(t) if r[0] == LOCAL_MISMATCH)
    if invalid:
        return RequestConsensus(generation, CacheDecision.PREFILL, 0, target, invalid)
    code, base = next(iter(proposals))
    return RequestConsensus(generation, _DECISIONS[code], base, target, ())


def resolve_boundary(rows: Iterable[Sequence[int]], stage: str) -> Tuple[int, int, int, int]:
    t = _table(rows, BOUNDARY_WORDS, (0, 1))
    bad = [i for i, r in enumerate(t) if not r[0]]
    if bad:
        raise CacheConsensusError(f"{stage} boundary rejected on ranks {bad}: {t}")
    if not _same(t, slice(1, None)):
        raise CacheConsensusError(f"{stage} boundary differs across ranks: {t}")
    generation, target, committed, pending = t[0][1:]
    if generation < 1 or target < 1 or committed != target or pending < 0:
        raise CacheConsensusError(f"invalid {stage} boundary: {t}")
    return generation, target, committed, pending


def resolve_retain(rows: Iterable[Sequence[int]]) -> Tuple[bool, Tuple[int, ...]]:
    t = _table(rows, BOUNDARY_WORDS, (0, 1))
    if not _same(t, slice(1, 3)):
        raise FatalTPInvariantError(f"restore generations / targets differ across ranks: {t}")
    rejected = tuple(i for i, r in enumerate(t) if not r[0])
    return not rejected, rejected


def resolve_failure(rows: Iterable[Sequence[int]]) -> Tuple[int, int, int, int]:
    t = _table(rows, BOUNDARY_WORDS, (0, 1))
    if any(r[0] != 1 for r in t):
        raise FatalTPInvariantError(f"failure is fatal on some rank: {t}")
    if not _same(t, slice(1, None)):
        raise FatalTPInvariantError(f"lifecycle differs across ranks during reset: {t}")
    return t[0][1], t[0][2], t[0][3], t[0][4]


def resolve_request_outcome(rows: Iterable[Sequence[int]]) -> Tuple[str, Tuple[int, int, int, int]]:
    t = _table(rows, BOUNDARY_WORDS, (0, 1, 2))
    if not _same(t, slice(1, None)):
        raise FatalTPInvariantError(f"lifecycle differs across ranks at request end: {t}")
    outcomes = {r[0] for r in t}
    life = (t[0][1], t[0][2], t[0][3], t[0][4])
    if outcomes == {2}:
        return "success", life
    if outcomes == {1}:
        return "reset", life
    raise FatalTPInvariantError(f"request outcome differs across ranks: {t}")


def all_gather_records(record: Sequence[int], group=None, device=None) -> List[Tuple[int, ...]]:
    """All-gather one row per rank (int64).  Single process: the row alone."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return [tuple(int(v) for v in record)]
    backend = dist.get_backend(group)
    dev = device if (device is not None and backend == "nccl") else ("cuda" if backend == "nccl" else "cpu")
    mine = torch.tensor(list(record), dtype=torch.int64, device=dev)
    out = torch.empty(dist.get_world_size(group) * mine.numel(), dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(out, mine, group=group)
    return [tuple(r) for r in out.view(-1, mine.numel()).tolist()]
