"""Host side of the LL packet channel (device side: ``csrc/ll.cuh``).

A channel is one symmetric inbox ``[2 halves][world][slots]`` of 8-byte packets plus two device
words shared by every channel of an engine: ``seq`` (the call sequence base that the last kernel
of each step advances) and ``status`` (sticky failure word).  All layers of an engine share one
channel, like the reference shares one reduce workspace per block type because multicast
objects are scarce (``nex_n2_5_pro/decode_engine.py:101-106``).

A context-parallel sub-channel is the same kind of inbox restricted to the ranks that share a
kv head (the reference's 4-rank ``cp_ctx``/``cp_lse`` channel, ``nex_n2_5_pro/attn_cp.py:76-174``).
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

from ..ops.lib import LLChannelStruct
from .symm import SymmetricBuffer

DEFAULT_BUDGET_MS = float(os.environ.get("NEXRT_WAIT_BUDGET_MS", "2000"))


class LLChannel:
    def __init__(
        self,
        device: torch.device,
        world: int,
        rank: int,
        slots: int,
        group=None,
        seq: Optional[torch.Tensor] = None,
        status: Optional[torch.Tensor] = None,
        budget_ms: float = DEFAULT_BUDGET_MS,
        members: Optional[Sequence[int]] = None,
    ):
        """``members``: global ranks forming this channel (default: the whole group).  The
        symmetric allocation is always made by the whole group; a sub-channel only uses the
        members' addresses and never the multicast alias."""
        self.device, self.slots = device, int(slots)
        self.members = list(members) if members is not None else list(range(world))
        self.world = len(self.members)
        self.rank = self.members.index(rank)
        self.seq = seq if seq is not None else torch.ones(1, dtype=torch.int32, device=device)
        self.status = status if status is not None else torch.zeros(1, dtype=torch.int32, device=device)
        nbytes = 2 * self.world * self.slots * 8
        self.buf = SymmetricBuffer(nbytes, device, group=group, world=world, rank=rank)
        s = LLChannelStruct()
        s.local = self.buf.local_ptr
        s.mc = self.buf.mc_ptr if (self.buf.mc_ptr and len(self.members) == world) else None
        for i in range(8):
            s.peer[i] = self.buf.peer_ptrs[self.members[i]] if i < self.world and world > 1 else None
        if world == 1:
            s.peer[0] = self.buf.local_ptr
        s.seq = self.seq.data_ptr()
        s.status = self.status.data_ptr()
        s.world, s.rank, s.slots, s.reserved = self.world, self.rank, self.slots, 0
        s.budget_ns = int(budget_ms * 1e6)
        self.struct = s

    @property
    def ref(self):
        return ctypes.byref(self.struct)

    @property
    def multicast(self) -> bool:
        return bool(self.struct.mc)

    def variant(self, multicast: bool = True, budget_ms: Optional[float] = None) -> LLChannelStruct:
        """A copy of the launch descriptor over the same inbox: without the multicast alias (one store per peer) and / or
        with another wait budget.  Benchmarks and tests use it to run both publishing forms in one process."""
        s = LLChannelStruct.from_buffer_copy(self.struct)
        if not multicast:
            s.mc = None
        if budget_ms is not None:
            s.budget_ns = int(budget_ms * 1e6)
        return s

    def set_budget_ms(self, ms: float) -> None:
        self.struct.budget_ns = int(ms * 1e6)

    def reset(self) -> None:
        """Zero the inbox and the failure word and restart the sequence.  Collective: every rank
        must call it at the same point, with nothing in flight (the caller barriers)."""
        self.buf.tensor.zero_()
        self.status.zero_()
        self.seq.fill_(1)
