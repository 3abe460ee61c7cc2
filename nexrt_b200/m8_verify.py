"""Eight-row target verify (with optional DFlash feature taps) on the decode engine.

API of the reference's ``M8Verify`` / ``M8CpVerify`` (``nex_n2_5_pro/m8_verify.py:205-1041``,
``nex_n2_5_pro/m8_cp.py:80-500``): ``run()``, ``capture()``, ``seed()``, ``reset_unit()``.  The state
rings of the engine are position indexed with one spare slot (9 state slots, 16 history slots for 8
rows), so a failed unit can be re-executed from the same base: ``reset_unit`` only clears the status
latches (reference m8_verify.py:722-741).
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from .decode_engine import DecodeEngine
from .runtime.control import Ctl, ring_no_alias

M = 8


class M8Verify:
    cp = False

    def __init__(self, engine: DecodeEngine):
        if engine.max_rows < M:
            raise ValueError("engine.max_rows must be >= 8")
        self.eng = engine
        gdn = [m for m in engine.mixers if hasattr(m, "state_ring_len")]
        if gdn and not ring_no_alias(M, gdn[0].conv_ring_len, gdn[0].state_ring_len):
            raise ValueError("state rings too small for an 8-row unit")

    def seed(self, verify_ids: Sequence[int]) -> None:
        """Host write of the 8 row ids of the next unit (ids[0] is the pending token)."""
        self.eng.set_rows(list(verify_ids))

    def run(self, end: bool = False, begin: bool = False) -> None:
        self.eng.step(M, cp=self.cp, end=end, begin=begin)

    def capture(self):
        return self.eng.capture(M, cp=self.cp)

    def reset_unit(self) -> None:
        """Clear the failure latches so that the same unit can run again (collective)."""
        eng = self.eng
        torch.cuda.synchronize(eng.dev)
        if eng.world > 1:
            dist.barrier(group=eng.group)
        eng.ctx.ctl[Ctl.STATUS] = 0
        eng.ctx.channel.buf.tensor.zero_()
        eng.ctx.seq.fill_(1)
        if eng.ctx.cp_channel is not None:
            eng.ctx.cp_channel.buf.tensor.zero_()
        torch.cuda.synchronize(eng.dev)
        if eng.world > 1:
            dist.barrier(group=eng.group)


    def guard_ok(self) -> bool:
        """No kernel of the unit wrote outside a scratch buffer it was handed.  Meaningful when the engine was built under
        ``NEXRT_CANARY=1`` (guard bands around every scratch buffer, ``runtime/audit.py``); without them there is nothing
        to check and the answer is True.  The reference guards its CP workspaces the same way
        (``nex_n2_5_pro/m8_cp.py:143-220,493-500``)."""
        return not self.eng.ctx.canaries_violated()


class M8CpVerify(M8Verify):
    cp = True

    def __init__(self, engine: DecodeEngine):
        super().__init__(engine)
        if not engine.cp:
            raise ValueError("the engine was built without the context-parallel arm")

    def cp_protocol_reset(self) -> None:
        """Resynchronise the context-parallel exchange after a round in which a rank of the kv group did not publish
        (collective, host side, never inside a capture).  The exchange carries no arrival counters - a packet is matched
        by the global call sequence in its tag - so resynchronising means: nothing in flight, every inbox of the group
        zero, the sequence restarted on every rank at once.  ``reset_unit`` already does that for both channels; this
        name exists for callers written against the reference's retry contract (``nex_n2_5_pro/m8_cp.py:328-431``)."""
        self.reset_unit()

    def cp_status_max(self) -> int:
        """Largest status word over the ranks (the CP waits latch into the engine's one status word)."""
        return self.eng.status_max()

    def cp_guard_ok(self) -> bool:
        return self.guard_ok()
