"""LM-head block: final norm + vocab-parallel GEMV + distributed top-k + sampler + commit.

Counterpart of the reference's ``Head`` (``nex_n2_5_pro/head.py:69-250``), whose four launches
(GEMV, per-rank top-k producer, 8-rank candidate reducer, sampler) are one kernel here; the
final-norm multiplier is applied to the activation, so the LM-head shard is used as stored (the
reference builds a fused ``W_fused = (1 + norm_w) x W`` copy, ``head.py:138-149``).
"""

from __future__ import annotations

from typing import Optional

import torch

from .ops.lib import check, ptr
from .runtime.context import StepContext
from .sampling import GREEDY, sampling_words

MODE_COMMIT = 1   # sample every row, prefix-accept, commit into the control block
MODE_DRAFT = 2    # greedy: row r's token goes to ctl ids[arg + r]


class Head:
    def __init__(self, ctx: StepContext, w: dict, init_sampling: bool = True):
        self.ctx, self.w = ctx, w
        self.logits: Optional[torch.Tensor] = None
        if init_sampling:
            self.set_sampling_config(0, *GREEDY)

    def set_sampling_config(self, seed, temperature, top_p, top_k) -> None:
        """Write the 64-byte sampling buffer in place (its address never moves)."""
        words = torch.tensor(sampling_words(seed, temperature, top_p, top_k), dtype=torch.int64)
        self.ctx.sampling.copy_(words.to(self.ctx.device))

    def enable_logits(self) -> torch.Tensor:
        """Also write the full fp32 logits of this rank's vocabulary rows (tests, golden checks)."""
        if self.logits is None:
            self.logits = torch.zeros(8, self.ctx.spec.vocab, dtype=torch.float32, device=self.ctx.device)
        return self.logits

    def forward(self, M: int = 1, mode: int = MODE_COMMIT, arg: int = 0, x: Optional[torch.Tensor] = None,
                ctl: Optional[torch.Tensor] = None) -> None:
        c, w = self.ctx, self.w
        cfg, spec = c.cfg, c.spec
        check(
            c.lib.nexrt_lmhead_sample(
                ptr(c.x if x is None else x), ptr(w["final_ln"]), ptr(w["lm_head"]), ptr(self.logits), ptr(c.head_cand), ptr(c.head_ticket),
                ptr(c.sampling), ptr(c.ctl if ctl is None else ctl), ptr(c.head_export), cfg.hidden, spec.vocab, spec.rank * spec.vocab, M, cfg.rms_eps, mode, arg,
                c.channel.ref, c.next_site(), c.n_cta, c.stream(),
            ),
            "lmhead_sample",
        )

    def sample_prefill(self, logits: torch.Tensor, position: int) -> None:
        """Sample the first token from full-vocabulary fp32 logits produced by a prefill
        (reference ``Head.sample_prefill``, head.py:237-250)."""
        c = self.ctx
        check(c.lib.nexrt_sample_logits(ptr(logits), ptr(c.sampling), ptr(c.ctl), logits.numel(), position, c.stream()), "sample_logits")
