"""Prefill bridge: chunked prefill driver with resume / suffix-extend and the ``Handoff`` facade.

In the reference the prompt is prefetched by SGLang and copied into the decode engine's dense caches
by device kernels (``Handoff.gather/append/finalize/scatter``, ``nex_n2_5_pro/sglang_prefill/
bridge.py:102-274``; ``chunked_prefill`` ``:310-398``).  Here prefill is the engine's own: it runs
the multi-row step kernels and writes KV rows, GDN states and the first token straight in decode
layout, so there is nothing to copy.  The same API is kept so that a serving loop written against
the reference keeps working: ``append`` records progress, ``finalize`` publishes the boundary and
clears the status latches, ``gather`` installs a saved state, ``scatter`` hands the state back.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Sequence, Tuple

from .cache_lifecycle import CacheBoundary

CP_THRESHOLD_BS1 = 48 * 1024          # reference bridge.py:50-52
DEFAULT_CHUNK = 8


@dataclass(frozen=True)
class PrefillSession:
    """The prompt state the engine currently holds: enough to extend it by an exact suffix."""

    tokens: Tuple[int, ...]
    first_token: int
    snapshot: object = None            # engine snapshot of the boundary (control block + GDN states)


def chunked_prefill(engine, tokens: Sequence[int], chunk: int = DEFAULT_CHUNK, on_chunk: Optional[Callable[[int, int, int], None]] = None,
                    resume: Optional[PrefillSession] = None, return_session: bool = False,
                    sample_next_token: Optional[Callable[[], int]] = None):
    """Prefill ``tokens`` in chunks of at most ``chunk`` rows.  With ``resume`` only the exact suffix
    after the session's tokens is evaluated.  ``on_chunk(start, end, next_token)`` runs after each
    chunk (``next_token`` is -1 for all but the last chunk, whose next token is the first generated
    token).  Returns ``first_token`` (and the new session)."""
    tokens = [int(t) for t in tokens]
    if not tokens:
        raise ValueError("prefill requires at least one token")
    if int(chunk) < 1:
        raise ValueError("chunk must be >= 1")
    start = 0
    if resume is not None:
        if not isinstance(resume, PrefillSession):
            raise TypeError("resume must be a PrefillSession")
        start = len(resume.tokens)
        if start > len(tokens) or tuple(tokens[:start]) != resume.tokens:
            raise ValueError("resume tokens are not an exact prefix of the new prompt")
        if resume.snapshot is not None:
            engine._restore(resume.snapshot)
    progress = []
    first = engine.prefill(tokens, chunk=int(chunk), resume_from=start, on_chunk=lambda s, e: progress.append((s, e)))
    if sample_next_token is not None:
        first = int(sample_next_token())
    if on_chunk is not None:
        for i, (s, e) in enumerate(progress):
            on_chunk(s, e, first if i == len(progress) - 1 else -1)
        if not progress:
            on_chunk(start, start, first)
    session = PrefillSession(tuple(tokens), int(first), engine._snapshot())
    return (first, session) if return_session else first


class Handoff:
    """API-compatible facade over the engine's state for callers written against the reference."""

    def __init__(self, engine):
        self.eng = engine
        self.appended = 0

    def gather(self, state: Dict) -> None:
        """Install a complete saved prefill state (reference ``gather``: whole-request fallback)."""
        self.eng.load_prefill(state)
        self.appended = int(state["L"])

    def append(self, start: int, end: int) -> None:
        """Rows ``[start, end)`` of the prompt are in the caches (they were written in place)."""
        if start != self.appended or end <= start:
            raise ValueError(f"append [{start}, {end}) does not continue {self.appended}")
        self.appended = end

    def finalize(self, first_token: Optional[int] = None) -> CacheBoundary:
        """Publish the decode boundary: pending token, committed length, cleared status latches."""
        import torch

        from ..runtime.control import Ctl

        ctl = self.eng.ctx.ctl
        if first_token is not None:
            ctl[Ctl.PENDING] = int(first_token)
            ctl[Ctl.IDS] = int(first_token)
        ctl[Ctl.STATUS] = 0
        torch.cuda.synchronize(self.eng.dev)
        w = ctl.tolist()
        return CacheBoundary(w[Ctl.COMMITTED_LEN], w[Ctl.PENDING], 0)

    def scatter(self) -> Dict:
        """Hand the current state back (multi-turn hand-back path of the reference)."""
        return self.eng.export_state()
