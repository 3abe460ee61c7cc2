"""MTP draft block: one round = two chained single-row drafts, the 4-row target verify, and the
draft layer's extend over the committed rows (which yields the first draft of the next round).

Counterpart of the reference's ``MtpDraft`` (``nex_n2_5_pro/mtp/block.py:84-583``: ``draft_phase``
``:518-522``, ``extend_phase`` ``:564-576``, ``round`` ``:579-583``).  The draft layer is an ordinary
gated-attention + MoE layer with its own KV cache; its passes reuse the engine's multi-row kernels
(no cloned translation units as in ``kernels/mtp/*``), take their base position and token ids from a
small control block of their own, and every pass is

    preprocess (embed + pre-fc norms, this rank's window of the concatenation)
    -> fc (FP8 GEMV + all-reduce, result replaces the residual rows)
    -> attention layer -> MoE -> [row select] -> LM head (greedy, token written into ids[k]).

Draft-layer position p pairs the target's hidden state of position p with token p+1, so after a
verify step that committed ``n`` tokens the extend pass covers positions ``C-n .. C-1`` and its last
row predicts the token after the pending one (draft 1); the two chained passes at positions C and
C+1 reuse the draft layer's own output hidden state (drafts 2 and 3).  Rows past the committed
length in the draft layer's KV cache are speculative and are overwritten by the next extend.
"""

from __future__ import annotations

import os
from typing import Dict, Optional, Sequence

import torch

from ..attn import FullAttn
from ..decode_engine import DecodeEngine
from ..head import MODE_DRAFT, Head
from ..moe import Moe
from ..ops.lib import check, ptr
from ..runtime.control import CTL_WORDS, Ctl

M_VERIFY = 4
PREP_EXTEND, PREP_DRAFT1, PREP_DRAFT2 = 0, 1, 2


class MtpDraft:
    def __init__(self, engine: DecodeEngine, w: Dict, cache_len: Optional[int] = None):
        if engine.max_rows < M_VERIFY:
            raise ValueError("the engine must be built with max_rows >= 4 for MTP")
        self.eng, self.w = engine, w
        c = self.ctx = engine.ctx
        dev = c.device
        lens = [m.cache_len for m in engine.mixers if isinstance(m, FullAttn)]
        self.attn = FullAttn(c, w["mixer"], cache_len=cache_len or (min(lens) if lens else c.cfg.cache_len))
        self.moe = Moe(c, w["moe"])
        self.head = Head(c, w["head"], init_sampling=False)
        self.dctl = torch.zeros(CTL_WORDS, dtype=torch.int32, device=dev)
        self.cat_win = torch.zeros(8, w["win"], dtype=torch.float32, device=dev)
        self.y_sel = torch.zeros(1, c.cfg.hidden, dtype=torch.bfloat16, device=dev)

    # ---- one pass of the draft layer over M rows (ids and base position are in self.dctl) ----------
    def _layer(self, M: int, hidden: torch.Tensor, hidden_row: int) -> None:
        c, w, lib, st = self.ctx, self.w, self.ctx.lib, self.ctx.stream()
        cfg = c.cfg
        check(
            lib.nexrt_mtp_preprocess(
                ptr(w["head"]["embed"]), ptr(self.dctl), ptr(hidden), ptr(w["ge"]), ptr(w["gf"]), ptr(w["gh"]), ptr(self.cat_win), cfg.hidden,
                cfg.vocab, w["win0"], w["win"], cfg.rms_eps, hidden_row, M, st,
            ),
            "mtp_preprocess",
        )
        check(
            lib.nexrt_oproj_allreduce(
                ptr(self.cat_win), None, None, ptr(w["fc_w"]), ptr(w["fc_s"]), ptr(c.x), cfg.hidden, w["win"], M, 0 | 4, cfg.rms_eps, 0,
                c.channel.ref, c.next_site(), None, 0, c.n_cta, st,
            ),
            "mtp_fc",
        )
        self.attn.forward(M, ctl=self.dctl)
        self.moe.forward(M)

    def _prep(self, mode: int, rows: int) -> None:
        c = self.ctx
        check(c.lib.nexrt_mtp_prep(ptr(c.ctl), ptr(self.dctl), mode, rows, c.stream()), "mtp_prep")

    def extend_phase(self, rows: int = M_VERIFY) -> None:
        """Draft layer over the rows the verify step just committed; leaves draft 1 in ids[1] and the
        hidden state of the last committed row in ``y_sel``."""
        c = self.ctx
        self._prep(PREP_EXTEND, rows)
        self._layer(rows, c.x, -1)
        check(c.lib.nexrt_row_select(ptr(c.x), ptr(self.dctl), ptr(self.y_sel), c.cfg.hidden, rows, c.stream()), "row_select")
        self.head.forward(1, mode=MODE_DRAFT, arg=1, x=self.y_sel)

    def draft_phase(self) -> None:
        """Two chained single-row passes: drafts 2 and 3 into ids[2], ids[3]."""
        c = self.ctx
        self._prep(PREP_DRAFT1, 1)
        self._layer(1, self.y_sel, 0)
        self.head.forward(1, mode=MODE_DRAFT, arg=2)
        self._prep(PREP_DRAFT2, 1)
        self._layer(1, c.x, 0)
        self.head.forward(1, mode=MODE_DRAFT, arg=3)

    def round(self, cp: bool = False) -> None:
        """One whole MTP round on the current stream (reference block.py:579-583)."""
        self.ctx.begin_step()
        self.draft_phase()
        self.eng.step(M_VERIFY, cp=cp, end=False, begin=False)
        self.extend_phase(M_VERIFY)
        self.eng.step_end()

    # ---- prefill ------------------------------------------------------------------------------------
    def _extend_wide(self, wp, ids: Sequence[int], n: int) -> None:
        """Target through wide chunks over ``ids[:n]``; after each chunk the draft layer extends over its rows, eight at
        a time: block ``k`` pairs the hidden rows of positions ``8k .. 8k+7`` with the tokens one position later (what
        ``_prep(PREP_EXTEND)`` derives from the control block after an 8-row step)."""
        eng, c = self.eng, self.ctx
        rows = 8
        table = torch.zeros(n // rows, CTL_WORDS, dtype=torch.int32)
        for k in range(n // rows):
            table[k, Ctl.COMMITTED_LEN] = k * rows
            table[k, Ctl.COMMIT_COUNT] = rows
            table[k, Ctl.IDS : Ctl.IDS + rows] = torch.tensor(ids[k * rows + 1 : k * rows + rows + 1], dtype=torch.int32)
        table = table.to(c.device)

        def after_chunk(start: int, x: torch.Tensor) -> None:
            for j in range(wp.T // rows):
                self.dctl.copy_(table[start // rows + j])
                c.begin_step()
                self._layer(rows, x[j * rows : (j + 1) * rows], -1)
                eng.step_end()

        wp.run(ids[:n], base=0, after_chunk=after_chunk)

    def prefill(self, ids: Sequence[int], chunk: int = 8, wide: Optional[int] = None) -> int:
        """Chunked prefill of target and draft layer together; returns the first generated token and
        leaves draft 1 ready for the first round.  ``wide`` (default: ``NEXRT_WIDE_PREFILL``, 0 = off): whole chunks of
        that many tokens go through the target's wide prefill path, the draft layer following eight rows at a time on
        the chunk's final hidden rows; the rest of the prompt takes the 8-row steps below."""
        eng, c = self.eng, self.ctx
        ids = [int(t) for t in ids]
        chunk = min(chunk, eng.max_rows)
        eng.reset(first_token=ids[0])
        pos = 0
        wide = int(os.environ.get("NEXRT_WIDE_PREFILL", "0") or 0) if wide is None else int(wide)
        if wide and len(ids) - 1 >= wide:
            wp = eng.wide_path(wide)
            if wp is not None:
                pos = (len(ids) - 1) // wide * wide
                self._extend_wide(wp, ids, pos)
        while pos < len(ids):
            n = min(chunk, len(ids) - pos)
            last = pos + n >= len(ids)
            eng.set_rows(ids[pos : pos + n])
            eng.set_forced_commit(n)
            c.begin_step()
            eng.step(n, end=False, begin=False)
            self._prep(PREP_EXTEND, n)
            if not last:  # the token after the chunk is the next prompt token, not the sampled one
                self.dctl[Ctl.IDS + n - 1 : Ctl.IDS + n] = torch.tensor([ids[pos + n]], dtype=torch.int32, device=c.device)
            self._layer(n, c.x, -1)
            if last:
                check(c.lib.nexrt_row_select(ptr(c.x), ptr(self.dctl), ptr(self.y_sel), c.cfg.hidden, n, c.stream()), "row_select")
                self.head.forward(1, mode=MODE_DRAFT, arg=1, x=self.y_sel)
            eng.step_end()
            pos += n
        eng.set_forced_commit(0)
        torch.cuda.synchronize(c.device)
        eng.mirror.resync()
        return int(c.ctl[Ctl.PENDING].item())
