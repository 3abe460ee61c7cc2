"""LM-head block: final norm + vocab-parallel GEMV + distributed top-k + sampler + commit.

Counterpart of the reference's ``Head`` (``nex_n2_5_pro/head.py:69-250``), whose four launches
(GEMV, per-rank top-k producer, 8-rank candidate reducer, sampler) are one kernel here; the
final-norm multiplier is applied to the activation, so the LM-head shard is used as stored (the
reference builds a fused ``W_fused = (1 + norm_w) x W`` copy, ``head.py:138-149``).
"""

from __future__ import annotations

import os

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
        self.wide_logits: Optional[torch.Tensor] = None
        self.tc_rows = int(os.environ.get("NEXRT_TC_HEAD_ROWS", "1")) or 1 << 30   # the logits GEMM pays off from one row (254 MB of bf16 weights per rank)
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
        if M >= self.tc_rows and cfg.hidden % 64 == 0 and cfg.hidden <= 4096 and spec.vocab % 2 == 0:
            # multi-row steps: logits of all rows in one tcgen05 GEMM (bf16 weights streamed once, hi + lo activation
            # planes), then the same top-k / exchange / sample / commit kernel reading those logits
            if self.wide_logits is None:
                self.wide_logits = torch.zeros(8, spec.vocab, dtype=torch.float32, device=c.device)
            lg = self.logits if self.logits is not None else self.wide_logits
            check(
                c.lib.nexrt_tc_router_logits(ptr(c.x if x is None else x), ptr(w["final_ln"]), ptr(w["lm_head"]), ptr(c.router_planes), ptr(lg),
                                             ptr(c.zero_ids), spec.vocab, spec.vocab, cfg.hidden, M, 1, cfg.rms_eps, None, ptr(c.status), c.stream()),
                "tc_lmhead_logits",
            )
            check(
                c.lib.nexrt_lmhead_sample_from_logits(
                    ptr(lg), ptr(c.head_cand), ptr(c.head_ticket), ptr(c.sampling), ptr(c.ctl if ctl is None else ctl), ptr(c.head_export), cfg.hidden,
                    spec.vocab, spec.rank * spec.vocab, M, mode, arg, c.channel.ref, c.next_site(), c.n_cta, c.stream(),
                ),
                "lmhead_sample_from_logits",
            )
            return
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
