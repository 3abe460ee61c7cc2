"""Gated full-attention layer block (non-CP and context-parallel arms).

Counterpart of the reference's ``FullAttn`` (``nex_n2_5_pro/attn.py:261-512``) and ``FullAttnCP``
(``nex_n2_5_pro/attn_cp.py:76-367``).  Three launches per layer: projection front (v appended to
the cache), split-KV decode (q/k norm + RoPE in its prologue, combine by the last CTA), and the
out-projection fused with the all-reduce and the residual.  In the context-parallel arm the
front also projects the q heads of the other ranks that share this rank's kv head (the
reference's duplicate-Q weights, ``attn.py:220-257``), the decode kernel attends only this
rank's window of the prefix and sends per-head partials to their owners, and the LSE merge runs
in the prologue of the out-projection kernel.

The bf16 KV cache is ``[kv_heads_local][cache_len][head_dim]`` for K and for V, pre-allocated for
the whole context (``attn.py:71-75,305-306``); ``cache_len`` may be shrunk for tests.
"""

from __future__ import annotations

import os

from typing import Optional

import torch

from .ops import wide
from .ops.lib import check, ptr
from .runtime.context import StepContext


class FullAttn:
    def __init__(self, ctx: StepContext, w: dict, cache_len: Optional[int] = None, cp_w: Optional[dict] = None):
        self.ctx, self.w, self.cp_w = ctx, w, cp_w
        cfg, spec, dev = ctx.cfg, ctx.spec, ctx.device
        self.cache_len = cache_len or cfg.cache_len
        shape = (spec.kv_heads, self.cache_len, cfg.head_dim)
        self.k_cache = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        self.v_cache = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        # rows from which the front projection runs as one tcgen05 GEMM (NEXRT_TC_ATTN_ROWS=0 switches it off)
        self.tc_rows = int(os.environ.get("NEXRT_TC_ATTN_ROWS", "8")) or 1 << 30   # no gain measured at 4 rows

    def reset(self) -> None:
        pass  # rows beyond committed_len are never read

    def forward(self, M: int = 1, cp: bool = False, ctl: Optional[torch.Tensor] = None) -> None:
        """``ctl``: control block whose committed length is the base position of the rows (default:
        the engine's; the MTP draft layer passes its own)."""
        c, lib = self.ctx, self.ctx.lib
        ctl = c.ctl if ctl is None else ctl
        cfg, spec, st = c.cfg, c.spec, c.stream()
        use_cp = cp and c.cp_channel is not None and self.cp_w is not None
        w = self.cp_w if use_cp else self.w
        nq = spec.q_heads * (spec.cp_size if use_cp else 1)
        R = (nq + spec.q_heads + 2 * spec.kv_heads) * cfg.head_dim
        if M >= self.tc_rows and R % 128 == 0 and cfg.hidden % 256 == 0 and cfg.hidden <= 4096:
            # multi-row steps: the q|gate|k|v projection of all rows is one tcgen05 GEMM, a tail kernel scatters it
            check(lib.nexrt_rows_norm_split(ptr(c.x), ptr(self.w["in_ln"]), ptr(c.moe_planes1), None, cfg.hidden, M, cfg.rms_eps, st), "rows_norm_split")
            check(lib.nexrt_tc_rows_gemm(ptr(w["front_w"]), ptr(w["front_s"]), ptr(c.moe_planes1), ptr(c.wide_pre), ptr(c.zero_ids), R, cfg.hidden, M,
                                         c.wide_ksplit, ptr(c.status), st), "tc_rows_gemm")
            check(lib.nexrt_attn_front_tail(ptr(c.wide_pre), ptr(ctl), ptr(c.q_raw), ptr(c.gate), ptr(c.k_raw), ptr(self.v_cache), cfg.head_dim, nq,
                                            spec.q_heads, spec.kv_heads, M, self.cache_len, c.wide_ksplit, st), "attn_front_tail")
        else:
            self._front_fused(M, w, nq, ctl)
        self._rest(M, use_cp, nq, ctl)

    def _front_fused(self, M, w, nq, ctl) -> None:
        c, lib = self.ctx, self.ctx.lib
        cfg, spec, st = c.cfg, c.spec, c.stream()
        check(
            lib.nexrt_attn_front(
                ptr(c.x), ptr(self.w["in_ln"]), ptr(w["front_w"]), ptr(w["front_s"]), ptr(ctl), ptr(c.q_raw), ptr(c.gate), ptr(c.k_raw),
                ptr(self.v_cache), cfg.hidden, cfg.head_dim, nq, spec.q_heads, spec.kv_heads, M, self.cache_len, cfg.rms_eps, c.n_cta, st,
            ),
            "attn_front",
        )

    def _rest(self, M, use_cp, nq, ctl) -> None:
        c, lib = self.ctx, self.ctx.lib
        cfg, spec, st = c.cfg, c.spec, c.stream()
        cp_site = c.next_site() if use_cp else 0
        # bit 8: the kernel may read the committed length before its dependency wait - true for the engine's own control
        # block inside a step (its only writer is the head at the end of the step, and the step's first kernel holds its
        # dependents back until everything before the step is complete), not for a draft layer's private block
        flags = 8 if (ctl is c.ctl and c.early_ctl) else 0
        check(
            lib.nexrt_attn_decode(
                ptr(c.q_raw), ptr(c.gate), ptr(c.k_raw), ptr(self.w["qn"]), ptr(self.w["kn"]), ptr(c.inv_freq), ptr(c.rope_table(self.cache_len)), ptr(ctl), ptr(self.k_cache),
                ptr(self.v_cache), ptr(c.ws_acc), ptr(c.ws_ml), ptr(c.attn_ticket), ptr(c.attn_out), cfg.head_dim, nq, spec.q_heads,
                spec.kv_heads, M, self.cache_len, cfg.rotary_dim, c.n_splits, cfg.rms_eps, flags, 0, 0, 0, spec.cp_size if use_cp else 1,
                spec.cp_rank if use_cp else 0, c.cp_channel.ref if use_cp else None, cp_site, st,
            ),
            "attn_decode",
        )
        n_cta = c.n_cta
        # the cluster form of the decode kernel has merged the context-parallel partials already (and gated them): the
        # out-projection then reads a plain input; the ticket form leaves the merge to the out-projection (mode 2)
        merge_here = use_cp and not lib.nexrt_attn_decode_merges_cp(c.n_splits)
        if wide.oproj_is_wide(c, spec.attn_local, M):
            wide.oproj_allreduce(c, c.attn_out, c.gate, None, self.w["out_w"], self.w["out_s"], spec.attn_local, M, 2 if merge_here else 0, cfg.head_dim,
                                 c.cp_channel.ref if merge_here else None, cp_site)
            return
        check(
            lib.nexrt_oproj_allreduce(
                ptr(c.attn_out), ptr(c.gate), None, ptr(self.w["out_w"]), ptr(self.w["out_s"]), ptr(c.x), cfg.hidden, spec.attn_local, M,
                2 if merge_here else 0, cfg.rms_eps, cfg.head_dim, c.ar_channel.ref, c.next_site(), c.cp_channel.ref if merge_here else None, cp_site,
                n_cta, st,
            ),
            "attn_oproj_allreduce",
        )
        c.after_allreduce(M)

    def load_kv(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """Install ``k, v [kv_heads_local][S][head_dim]`` (already normalised and rotated)."""
        S = k.shape[1]
        self.k_cache[:, :S] = k.to(self.k_cache)
        self.v_cache[:, :S] = v.to(self.v_cache)
