"""DFlash block draft: 8 proposals per round from a small dense BF16 stack conditioned on target
features, verified by the target in one 8-row step.

Counterpart of the reference's ``DFlashBlock`` (``nex_n2_5_pro/dflash/block.py:152-692``;
``round`` ``:593-675``).  One round on the device:

    context phase   features of the rows the last verify committed (taps of 8 target layers,
                    concatenated) -> fc (+ all-reduce) -> per draft layer k/v projection of those
                    context rows, published into the draft's KV cache at their positions
    draft phase     rows = [embed(pending), embed(mask) x 7] -> 6 x { qkv, publish block k/v,
                    attention (the 8 rows see each other and the context; sliding window on 5 layers),
                    o-proj + all-reduce, gate/up, down + all-reduce } -> final norm + shared LM head
                    (greedy) -> proposals become ids[1..7]
    verify          the engine's 8-row step with feature taps

The draft's attention takes its base position from the draft's own control block, so the captured
graph is independent of the request (the reference re-captures per request because its draft
attention bakes the base position, ``dflash/serve.py:29-45``).
"""

from __future__ import annotations

import os
from typing import Dict, Optional, Sequence

import torch

from ..decode_engine import DecodeEngine
from ..head import MODE_DRAFT, Head
from ..ops.lib import check, ptr
from ..runtime.control import CTL_WORDS, Ctl
from .config import DFlashConfig

M8 = 8


class DFlashBlock:
    def __init__(self, engine: DecodeEngine, dc: DFlashConfig, w: Dict, cache_len: Optional[int] = None):
        if engine.max_rows < M8:
            raise ValueError("the engine must be built with max_rows >= 8 for DFlash")
        dc.validate_kernel_contract(engine.cfg, engine.world)
        self.eng, self.dc, self.w = engine, dc, w
        c = self.ctx = engine.ctx
        dev, H, hd = c.device, dc.hidden, dc.head_dim
        self.q, self.kv, self.I = w["q_local"], w["kv_local"], w["I_local"]
        self.cache_len = cache_len or engine._kv_budget()
        z = lambda *s, dtype=torch.float32: torch.zeros(*s, dtype=dtype, device=dev)
        self.k_cache = [z(self.kv, self.cache_len, hd, dtype=torch.bfloat16) for _ in range(dc.n_layers)]
        self.v_cache = [z(self.kv, self.cache_len, hd, dtype=torch.bfloat16) for _ in range(dc.n_layers)]
        self.dctl = z(CTL_WORDS, dtype=torch.int32)     # draft rows: base position = committed length
        self.cctl = z(CTL_WORDS, dtype=torch.int32)     # context rows: base position = committed length - commit count
        self.context = z(M8, H, dtype=torch.bfloat16)
        self.R = (self.q + 2 * self.kv) * hd
        self.qkv = z(M8, self.R)
        self.ckv = z(M8, 2 * self.kv * hd)
        self.attn_out = z(M8, self.q * hd)
        self.gu = z(M8, 2 * self.I)
        G = self.q // self.kv
        self.n_splits = max(1, c.n_cta // self.kv)
        self.ws_acc = z(self.kv, self.n_splits, M8 * G, hd)
        self.ws_ml = z(self.kv, self.n_splits, M8 * G, 2)
        self.ticket = z(self.kv, dtype=torch.int32)
        inv = 1.0 / (dc.rope_theta ** (torch.arange(0, dc.rotary_dim, 2, dtype=torch.float32) / dc.rotary_dim))
        self.inv_freq = inv.to(dev)
        ang = torch.arange(self.cache_len, dtype=torch.float32, device=dev)[:, None] * self.inv_freq[None, :]
        self.rope = torch.stack([torch.cos(ang), torch.sin(ang)], -1).contiguous()
        self.taps = engine.enable_taps(dc.target_layer_ids)
        self.head = Head(c, {"final_ln": w["final_ln"], "lm_head": engine.head.w["lm_head"]}, init_sampling=False)
        self.embed = engine.embed

    def _dense(self, inp, gamma, wt, out, x, R, K, M, in_mode, out_mode, ld_in=0):
        c = self.ctx
        site = c.next_site() if out_mode else 0
        check(c.lib.nexrt_dense_bf16(ptr(inp), ptr(gamma), ptr(wt), ptr(out), ptr(x), R, K, M, in_mode, out_mode, ld_in, self.dc.rms_eps,
                                     c.channel.ref, site, c.stream()), "dense_bf16")

    def _publish(self, kv, ld, k_off, v_off, kn, ctl, layer, M):
        c, dc = self.ctx, self.dc
        check(c.lib.nexrt_kv_publish(ptr(kv), ld, k_off, v_off, ptr(kn), ptr(self.rope), ptr(ctl), ptr(self.k_cache[layer]),
                                     ptr(self.v_cache[layer]), dc.head_dim, self.kv, M, self.cache_len, dc.rotary_dim, dc.rms_eps, 0,
                                     c.stream()), "kv_publish")

    # ---- context rows: features of committed positions -> draft KV caches ---------------------------
    def context_phase(self, M: int = M8, prep: bool = True) -> None:
        c, dc, w, H, hd = self.ctx, self.dc, self.w, self.dc.hidden, self.dc.head_dim
        if prep:
            check(c.lib.nexrt_mtp_prep(ptr(c.ctl), ptr(self.cctl), 0, M, c.stream()), "dflash_prep")
        # fc over this rank's window of the concatenated taps, all-reduced into the context rows
        self._dense(self.taps[:, w["win0"] :], None, w["fc"], None, self.context, H, w["win"], M, 3, 2, ld_in=self.taps.shape[1])
        for l, lw in enumerate(w["layers"]):
            self._dense(self.context, w["hidden_ln"], lw["wkv"], self.ckv, None, 2 * self.kv * hd, H, M, 0, 0)
            self._publish(self.ckv, 2 * self.kv * hd, 0, self.kv * hd, lw["kn"], self.cctl, l, M)

    # ---- the 8 draft rows ------------------------------------------------------------------------------
    def draft_phase(self) -> None:
        c, dc, w, H, hd = self.ctx, self.dc, self.w, self.dc.hidden, self.dc.head_dim
        st = c.stream
        check(c.lib.nexrt_dflash_noise(ptr(self.embed), ptr(c.ctl), ptr(c.x), ptr(self.dctl), H, dc.vocab, dc.mask_token_id, M8, st()), "noise")
        for l, lw in enumerate(w["layers"]):
            self._dense(c.x, lw["in_ln"], lw["wqkv"], self.qkv, None, self.R, H, M8, 0, 0)
            self._publish(self.qkv, self.R, self.q * hd, (self.q + self.kv) * hd, lw["kn"], self.dctl, l, M8)
            k_raw = self.qkv[:, self.q * hd :]
            check(
                c.lib.nexrt_attn_decode(
                    ptr(self.qkv), ptr(self.qkv), ptr(k_raw), ptr(lw["qn"]), ptr(lw["kn"]), ptr(self.inv_freq), ptr(self.rope), ptr(self.dctl),
                    ptr(self.k_cache[l]), ptr(self.v_cache[l]), ptr(self.ws_acc), ptr(self.ws_ml), ptr(self.ticket), ptr(self.attn_out), hd,
                    self.q, self.q, self.kv, M8, self.cache_len, dc.rotary_dim, self.n_splits, dc.rms_eps, 3, lw["window"], self.R, self.R,
                    1, 0, None, 0, st(),
                ),
                "dflash_attn",
            )
            self._dense(self.attn_out, None, lw["wo"], None, c.x, H, self.q * hd, M8, 1, 1)
            self._dense(c.x, lw["post_ln"], lw["wgu"], self.gu, None, 2 * self.I, H, M8, 0, 0)
            self._dense(self.gu, None, lw["wdown"], None, c.x, H, self.I, M8, 2, 1)
        self.head.forward(M8, mode=MODE_DRAFT, arg=0, ctl=self.dctl)
        check(c.lib.nexrt_dflash_commit(ptr(c.ctl), ptr(self.dctl), M8, st()), "dflash_commit")

    def round(self, cp: bool = False) -> None:
        self.ctx.begin_step()
        self.context_phase()
        self.draft_phase()
        self.eng.step(M8, cp=cp, end=False, begin=False)
        self.eng.step_end()

    # ---- prefill -------------------------------------------------------------------------------------
    def prefill(self, ids: Sequence[int], wide: Optional[int] = None) -> int:
        """Chunked prefill of the target (8-row steps with taps) and of the draft's context caches.  ``wide`` (default:
        ``NEXRT_WIDE_PREFILL``, 0 = off): whole chunks of that many tokens go through the target's wide prefill path,
        which also records the taps of its rows; the context phase follows eight rows at a time."""
        eng, c = self.eng, self.ctx
        ids = [int(t) for t in ids]
        eng.reset(first_token=ids[0])
        pos = 0
        wide = int(os.environ.get("NEXRT_WIDE_PREFILL", "0") or 0) if wide is None else int(wide)
        if wide and len(ids) - 1 >= wide:
            wp = eng.wide_path(wide)
            if wp is not None:
                pos = (len(ids) - 1) // wide * wide

                def after_chunk(start: int, x: torch.Tensor) -> None:
                    for j in range(wp.T // M8):
                        self.taps.copy_(wp.taps[j * M8 : (j + 1) * M8])
                        self.cctl.zero_()
                        self.cctl[Ctl.COMMITTED_LEN] = start + j * M8      # positions of the eight context rows
                        self.cctl[Ctl.COMMIT_COUNT] = M8
                        c.begin_step()
                        self.context_phase(M8, prep=False)
                        eng.step_end()

                wp.run(ids[:pos], base=0, after_chunk=after_chunk)
        while pos < len(ids):
            n = min(M8, len(ids) - pos)
            eng.set_rows(ids[pos : pos + n])
            eng.set_forced_commit(n)
            c.begin_step()
            eng.step(n, end=False, begin=False)
            self.context_phase(n)
            eng.step_end()
            pos += n
        eng.set_forced_commit(0)
        # the last prefill step left no fresh commit for the first round's context phase
        c.ctl[Ctl.COMMIT_COUNT] = 0
        torch.cuda.synchronize(c.device)
        eng.mirror.resync()
        return int(c.ctl[Ctl.PENDING].item())
