"""Host model of the LL packet protocol (``csrc/ll.cuh``) for protocol tests without GPUs.

Each rank is a thread.  A rank's inbox is ``[2 halves][world][slots]`` of ``(tag, payload)`` pairs written as one
unit (the device writes them with one 8-byte store); ``seq`` is the call-sequence base a rank advances at the end of
every "graph" by that graph's number of channel users, exactly as ``step_end_kernel`` does.  A call is

    g = seq + site;  tag = g | 0x8000_0000;  half = g & 1
    publish (tag, own) into slot idx of region [half][rank] of every peer's inbox
    poll the own inbox's region [half][src] for every src until its tag matches (bounded), add in rank order

The model keeps the properties the kernels rely on and lets a test break them on purpose (a rank that never sends, a
mix of graphs with different site counts, ranks that run at different speeds):

* a packet of an older call can never be taken for the current one, because the tag is the call number;
* consecutive calls alternate halves, and a peer can be at most one call ahead of the slowest rank (it needs that
  rank's packet to finish its own call), so a region is never overwritten while a rank may still have to read it;
* a wait gives up after its budget, latches the sticky status and reads the missing value as zero.
"""

from __future__ import annotations

import random
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

STATUS_OK, STATUS_REDUCE_TIMEOUT = 0, 1


@dataclass
class RankState:
    rank: int
    world: int
    slots: int
    inbox: list = field(default_factory=list)      # [half][src][slot] -> (tag, payload)
    seq: int = 1
    status: int = STATUS_OK
    stale_reads: int = 0                           # packets seen with a tag that is not the awaited one (never consumed)

    def __post_init__(self):
        self.inbox = [[[(0, 0.0)] * self.slots for _ in range(self.world)] for _ in range(2)]


class LLModel:
    def __init__(self, world: int, slots: int, budget_s: float = 2.0, silent: Sequence[int] = ()):
        self.world, self.slots, self.budget_s = world, slots, budget_s
        self.ranks = [RankState(r, world, slots) for r in range(world)]
        self.silent = set(silent)                  # ranks whose stores never leave (a peer that never joins)

    # ---- device-side primitives -----------------------------------------------------------------------
    def begin(self, me: RankState, site: int):
        g = (me.seq + site) & 0xFFFFFFFF
        return g | 0x80000000, g & 1

    def publish(self, me: RankState, tag: int, half: int, idx: int, payload: float) -> None:
        if me.rank in self.silent:
            return
        for peer in self.ranks:
            if peer.rank != me.rank:
                peer.inbox[half][me.rank][idx] = (tag, payload)     # one tuple assignment == one 8-byte store

    def wait(self, me: RankState, tag: int, half: int, src: int, idx: int) -> Optional[float]:
        deadline = None
        failed = me.status != STATUS_OK
        while True:
            t, v = me.inbox[half][src][idx]
            if t == tag:
                return v
            if t != 0:
                me.stale_reads += 1
            if failed:
                return None
            if deadline is None:
                deadline = time.monotonic() + self.budget_s
            elif time.monotonic() > deadline:
                me.status = me.status or STATUS_REDUCE_TIMEOUT
                return None
            time.sleep(0)

    def allreduce(self, me: RankState, site: int, idx: int, own: float) -> float:
        """``ll_allreduce_f32``: publish, then add the world's values in rank order (own value from the register)."""
        if self.world == 1:
            return own
        tag, half = self.begin(me, site)
        self.publish(me, tag, half, idx, own)
        total = 0.0
        for src in range(self.world):
            if src == me.rank:
                total += own
            else:
                v = self.wait(me, tag, half, src, idx)
                total += 0.0 if v is None else v
        return total

    def end_graph(self, me: RankState, n_sites: int) -> None:
        me.seq = (me.seq + n_sites) & 0xFFFFFFFF

    # ---- driver ---------------------------------------------------------------------------------------------
    def run(self, program: Callable[["LLModel", RankState], List[float]], jitter_s: float = 0.0, seed: int = 0) -> List[List[float]]:
        """Run ``program(model, rank_state)`` on one thread per rank; returns the per-rank result lists."""
        out: List[Optional[List[float]]] = [None] * self.world
        errors: List[BaseException] = []

        def body(r: int) -> None:
            rng = random.Random(seed * 131 + r)
            me = self.ranks[r]
            me._sleep = (lambda: time.sleep(rng.random() * jitter_s)) if jitter_s else (lambda: None)
            try:
                out[r] = program(self, me)
            except BaseException as e:  # noqa: BLE001
                errors.append(e)

        threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(self.world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(60)
        if errors:
            raise errors[0]
        return out  # type: ignore[return-value]
