"""Four-row target verify on the decode engine's own weights, caches and kernels.

API of the reference's ``M4VerifyNonCP`` / ``M4VerifyCp`` (``nex_n2_5_pro/m4_verify.py:155-1227``):
``run()`` launches the 4-row verify chain (embed of ``ids[0..3]``, every layer, LM head, sampling,
prefix accept and commit), ``forced_commit`` pins the number of committed tokens for fixed-acceptance
benchmarks, and the CP arm switches the attention layers to their context-parallel form above
``CP_THRESHOLD_M4`` tokens.  No lane-major weight prepacks, history rings or LL wires are owned here:
the engine's kernels take the row count at run time and its rings are position indexed for every
mode, so the verifier is a view of the engine rather than a second copy of it.
"""

from __future__ import annotations

from .decode_engine import DecodeEngine
from .runtime.control import Ctl

M = 4
CP_THRESHOLD_M4 = 229_376   # reference m4_verify.py:66-69


class M4VerifyNonCP:
    cp = False

    def __init__(self, engine: DecodeEngine):
        if engine.max_rows < M:
            raise ValueError("engine.max_rows must be >= 4")
        self.eng = engine

    def run(self, end: bool = False, begin: bool = False) -> None:
        self.eng.step(M, cp=self.cp, end=end, begin=begin)

    @property
    def forced_commit(self) -> int:
        return int(self.eng.ctx.ctl[Ctl.FORCED_COMMIT].item())

    @forced_commit.setter
    def forced_commit(self, count: int) -> None:
        self.eng.set_forced_commit(int(count))

    def set_forced_schedule(self, seed: int, mean_accept: float) -> None:
        """Seeded commit-count schedule with the given mean (fixed-acceptance benchmarking)."""
        self.eng.set_forced_commit(0, seed=seed, mean10=int(round(mean_accept * 10)))

    def load(self, verify_ids) -> None:
        self.eng.set_rows(list(verify_ids))


class M4VerifyCp(M4VerifyNonCP):
    cp = True

    def __init__(self, engine: DecodeEngine):
        super().__init__(engine)
        if not engine.cp:
            raise ValueError("the engine was built without the context-parallel arm")


M4Verify = M4VerifyNonCP
