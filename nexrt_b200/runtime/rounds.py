"""Host side of a speculative request: replay the round graph, read each round's result from the host mirror, stop.

The MTP and the DFlash request loops are the same loop (reference ``nex_n2_5_pro/mtp/serve.py:83-187`` and
``nex_n2_5_pro/dflash/serve.py``): one round is in flight while the previous one is read, a round commits between one
token and the verify width, and the request ends at a stop token, at ``max_new`` tokens or where the caches end.  Nothing
here touches the device except ``graph.replay()``, so the loop is tested on the CPU with a scripted mirror
(``tests/test_rounds_cpu.py``).
"""

from __future__ import annotations

from typing import Callable, FrozenSet, Iterable, List, Optional, Union

from .control import Ctl

Stops = Union[None, int, Iterable[int]]


def stop_set(eos: Stops) -> FrozenSet[int]:
    """The ``eos`` argument of the generate loops as a set: ``None`` (never stop), one token id, or any iterable of ids
    (a model's generation config and its tokenizer may each name several).  Negative ids never match a token."""
    if eos is None:
        return frozenset()
    if isinstance(eos, bool):
        raise TypeError("eos must be a token id or an iterable of token ids")
    if isinstance(eos, int):
        return frozenset((eos,)) if eos >= 0 else frozenset()
    return frozenset(int(t) for t in eos if t is not None and int(t) >= 0)


def consume_rounds(eng, graph, max_new: int, eos: Stops = None, on_tokens: Optional[Callable[[List[int]], None]] = None,
                   stats: Optional[dict] = None, reserve: int = 0, what: str = "round") -> List[int]:
    """Replay ``graph`` (one speculative round of ``eng``) until ``max_new`` tokens are out, a stop token is emitted or the
    committed length comes within ``reserve`` rows of the cache end.  Returns the emitted tokens, the stop token included;
    ``on_tokens`` sees exactly those tokens, round by round; ``stats`` receives ``rounds`` and ``accept_mean`` (tokens
    committed per round, whether or not the request kept them).  A round that latched a status or committed nothing ends
    the request with ``RuntimeError`` after the rounds already in flight have been waited for."""
    stops = stop_set(eos)
    eng.mirror.resync()
    out: List[int] = []
    budget = eng._kv_budget() - reserve
    rounds = accepted = 0

    def launch() -> int:
        graph.replay()
        return eng.mirror.next_gen()

    def drain(pending: List[int]) -> None:
        for gen in pending:
            eng.mirror.wait(gen)

    pending = [launch()] if max_new > 0 else []
    while pending:
        if len(pending) < 2 and len(out) + len(pending) < max_new:      # every round commits at least one token
            pending.append(launch())
        words = eng.mirror.wait(pending.pop(0))
        if words[Ctl.STATUS] != 0 or words[Ctl.COMMIT_COUNT] <= 0:
            drain(pending)
            raise RuntimeError(f"{what} failed: status {words[Ctl.STATUS]}")
        n = words[Ctl.COMMIT_COUNT]
        toks = list(words[Ctl.EMITTED : Ctl.EMITTED + n])
        rounds += 1
        accepted += n
        kept, stop = 0, False
        for t in toks:
            out.append(t)
            kept += 1
            if t in stops or len(out) >= max_new:
                stop = True
                break
        if on_tokens and kept:
            on_tokens(toks[:kept])
        if stop or words[Ctl.COMMITTED_LEN] >= budget:
            drain(pending)
            break
    if stats is not None:
        stats.update(rounds=rounds, accept_mean=accepted / max(rounds, 1))
    return out
