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


class BlockModel(LLModel):
    """Host model of the block protocol of the wide prefill's all-reduce (``csrc/prefill.cu:
    planes_allreduce_residual_kernel``) over the same inbox, sequence word and status as the packet protocol.

    A region ``[half][src]`` holds ``ctas * width`` data values followed by one flag word per CTA.  CTA ``b`` of a rank
    stores its ``width`` values untagged into region ``[half][own rank]`` of every peer, then the call's tag into flag
    ``b`` of that region (the device orders the two with a system fence and a barrier; here the flag is simply written
    last); it polls flag ``b`` of every peer region of its own inbox and only then reads that region's values.  Data
    carries no tag, so nothing but the ordering of calls keeps a region from being overwritten before it was read:

    * the CTAs of one call of one rank may run in any order and side by side, but call ``k + 1`` of a rank starts only
      after ALL its CTAs of call ``k`` have finished (stream order; programmatic launches wait for the whole grid);
    * CTA ``b`` of call ``k + 1`` finishes only once it saw every peer's flag ``b`` of call ``k + 1``, so a rank that is
      through call ``k + 1`` proves every peer through call ``k``; its stores of call ``k + 2`` (the same half as ``k``)
      then land in regions nobody reads any more.

    Because CTA ``b`` waits for CTA ``b`` of every peer, the CTAs of a call must either all be resident or be dispatched
    in the same (index) order on every rank; both hold on the device (grids of at most 1024 CTAs, dispatched in order).

    ``stale_data`` counts values a CTA read that were not the ones its peer wrote for the awaited call (the payload of
    the model encodes (call, rank, cta, lane), which the device's data does not need to)."""

    def __init__(self, world: int, ctas: int, width: int, budget_s: float = 2.0, silent: Sequence[int] = ()):
        super().__init__(world, ctas * width + ctas, budget_s, silent)
        self.ctas, self.width = ctas, width
        self.stale_data = [0] * world

    def cta(self, me: RankState, site: int, b: int, own: List[float], expect: Optional[Callable[[int], List[float]]] = None) -> List[float]:
        """One CTA of one call: returns the rank-ordered sums of its ``width`` values (missing peers count as zero)."""
        tag, half = self.begin(me, site)
        lo, flag = b * self.width, self.ctas * self.width + b
        if me.rank not in self.silent:
            for peer in self.ranks:
                if peer.rank != me.rank:
                    region = peer.inbox[half][me.rank]
                    for j, v in enumerate(own):
                        region[lo + j] = (0, v)                  # plain data: no tag travels with it
                    region[flag] = (tag, 0.0)                    # published after the data
        total = [0.0] * self.width
        for src in range(self.world):
            if src == me.rank:
                vals: Optional[List[float]] = own
            elif self.wait(me, tag, half, src, flag) is None:
                vals = None
            else:
                vals = [me.inbox[half][src][lo + j][1] for j in range(self.width)]
                if expect is not None and vals != expect(src):
                    self.stale_data[me.rank] += 1
            if vals is not None:
                total = [t + v for t, v in zip(total, vals)]
        return total

    def call(self, me: RankState, site: int, own_of: Callable[[int], List[float]], expect_of=None, order: Optional[Sequence[int]] = None,
             parallel: bool = False) -> List[List[float]]:
        """All CTAs of one call of rank ``me``: in ``order`` one after the other, or side by side on threads; the call
        returns when every CTA has finished (the kernel boundary)."""
        order = list(range(self.ctas)) if order is None else list(order)
        out: List[Optional[List[float]]] = [None] * self.ctas

        def one(b: int) -> None:
            out[b] = self.cta(me, site, b, own_of(b), None if expect_of is None else (lambda src: expect_of(src, b)))

        if parallel:
            ts = [threading.Thread(target=one, args=(b,), daemon=True) for b in order]
            for t in ts:
                t.start()
            for t in ts:
                t.join(60)
        else:
            for b in order:
                one(b)
        return out  # type: ignore[return-value]
