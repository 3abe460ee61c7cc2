"""Gated-delta-net (linear attention) layer block: weights, per-layer rings, launch sequence.

Counterpart of the reference's ``Gdn`` (``nex_n2_5_pro/gdn.py:142-250``): three launches per
layer, front -> recurrence -> out-projection fused with the tensor-parallel all-reduce and the
residual add.  Differences: 1..8 token rows through the same kernels; the conv history and the
recurrent state live in position-indexed rings (``conv_ring [R_c][C]``, ``state_ring
[R_s][nv][128][128]``) for every mode; the input RMSNorm multiplier is applied in the kernel
instead of being folded into re-quantised weights (``gdn.py:83-113``).
"""

from __future__ import annotations

import torch

import os

from .ops import wide
from .ops.lib import check, ptr
from .runtime.context import StepContext


class Gdn:
    def __init__(self, ctx: StepContext, w: dict, state_ring: int = 2, conv_ring: int = 16):
        self.ctx, self.w = ctx, w
        spec, dev = ctx.spec, ctx.device
        self.state_ring_len, self.conv_ring_len = state_ring, conv_ring
        ba = w["ba_w"]
        self.ba_rows_pad = (ba.shape[0] + 15) // 16 * 16   # zero rows up to a whole 16-row tensor-core tile
        if "ba_w_pad" not in w:
            pad = torch.zeros(self.ba_rows_pad, ba.shape[1], dtype=ba.dtype, device=ba.device)
            pad[: ba.shape[0]] = ba
            w["ba_w_pad"] = pad
        # rows from which the front projection runs as one tcgen05 GEMM (NEXRT_TC_ROWS=0 switches it off)
        self.tc_rows = int(os.environ.get("NEXRT_TC_ROWS", "4")) or 1 << 30
        self.tc_ok = spec.gdn_front_rows % 128 == 0 and ctx.cfg.hidden % 256 == 0 and ctx.cfg.hidden <= 4096
        self.conv_ring = torch.zeros(conv_ring, spec.gdn_qkv_rows, dtype=torch.float32, device=dev)
        self.state_ring = torch.zeros(state_ring, spec.gdn_v, 128, 128, dtype=torch.float32, device=dev)

    def reset(self) -> None:
        self.conv_ring.zero_()
        self.state_ring.zero_()

    def forward(self, M: int = 1) -> None:
        c, w, lib = self.ctx, self.w, self.ctx.lib
        cfg, spec, st = c.cfg, c.spec, c.stream()
        if M >= self.tc_rows and self.tc_ok:
            # multi-row steps: the q|k|v|z projection of all rows is one tcgen05 GEMM (weights streamed once),
            # then a small tail kernel does the conv ring, SiLU, z store and the b/a rows
            R = spec.gdn_front_rows
            check(lib.nexrt_rows_norm_split(ptr(c.x), ptr(w["in_ln"]), ptr(c.moe_planes1), ptr(c.wide_xn), cfg.hidden, M, cfg.rms_eps, st), "rows_norm_split")
            check(lib.nexrt_tc_rows_gemm(ptr(w["front_w"]), ptr(w["front_s"]), ptr(c.moe_planes1), ptr(c.wide_pre), ptr(c.zero_ids), R, cfg.hidden, M,
                                         c.wide_ksplit, ptr(c.status), st), "tc_rows_gemm")
            check(
                lib.nexrt_gdn_front_tail(
                    ptr(c.wide_pre), ptr(c.wide_xn), ptr(w["ba_w_pad"]), ptr(w["conv_w"]), ptr(w["a_log"]), ptr(w["dt_bias"]), ptr(c.ctl),
                    ptr(self.conv_ring), ptr(c.gdn_qkv), ptr(c.gdn_z), ptr(c.gdn_beta), ptr(c.gdn_g), cfg.hidden, R, spec.gdn_qkv_rows, spec.gdn_v, M,
                    self.conv_ring_len, c.wide_ksplit, st,
                ),
                "gdn_front_tail",
            )
        else:
            self._front_fused(M)
        self._rest(M)

    def _front_fused(self, M: int) -> None:
        c, w, lib = self.ctx, self.w, self.ctx.lib
        cfg, spec, st = c.cfg, c.spec, c.stream()
        check(
            lib.nexrt_gdn_front(
                ptr(c.x), ptr(w["in_ln"]), ptr(w["front_w"]), ptr(w["front_s"]), ptr(w["ba_w_pad"]), ptr(w["conv_w"]), ptr(w["a_log"]),
                ptr(w["dt_bias"]), ptr(c.ctl), ptr(self.conv_ring), ptr(c.gdn_qkv), ptr(c.gdn_z), ptr(c.gdn_beta), ptr(c.gdn_g),
                cfg.hidden, spec.gdn_front_rows, spec.gdn_qkv_rows, spec.gdn_v, M, self.conv_ring_len, cfg.rms_eps, self.ba_rows_pad, c.n_cta, st,
            ),
            "gdn_front",
        )

    def _rest(self, M: int) -> None:
        c, w, lib = self.ctx, self.w, self.ctx.lib
        cfg, spec, st = c.cfg, c.spec, c.stream()
        check(
            lib.nexrt_gdn_core(
                ptr(c.gdn_qkv), ptr(c.gdn_beta), ptr(c.gdn_g), ptr(c.ctl), ptr(self.state_ring), ptr(c.gdn_out), spec.gdn_qk, spec.gdn_v,
                M, self.state_ring_len, spec.gdn_qkv_rows, st,
            ),
            "gdn_core",
        )
        n_cta = c.n_cta
        if wide.oproj_is_wide(c, spec.gdn_local, M):
            wide.oproj_allreduce(c, c.gdn_out, c.gdn_z, w["gnorm_w"], w["out_w"], w["out_s"], spec.gdn_local, M, 1, 128, None, 0)
            return
        check(
            lib.nexrt_oproj_allreduce(
                ptr(c.gdn_out), ptr(c.gdn_z), ptr(w["gnorm_w"]), ptr(w["out_w"]), ptr(w["out_s"]), ptr(c.x), cfg.hidden, spec.gdn_local,
                M, 1, cfg.rms_eps, 128, c.ar_channel.ref, c.next_site(), None, 0, n_cta, st,
            ),
            "gdn_oproj_allreduce",
        )
        c.after_allreduce(M)

    # ---- state hand-off (prefill states, tests) ------------------------------------------------
    def load_state(self, position: int, conv_tail: torch.Tensor, state: torch.Tensor) -> None:
        """Install the state after ``position`` tokens: ``conv_tail [C,3]`` = pre-conv rows of the
        last three positions (oldest first), ``state [nv,128(k),128(v)]``."""
        self.reset()
        for j in range(3):
            p = position - 3 + j
            if p >= 0:
                self.conv_ring[p % self.conv_ring_len] = conv_tail[:, j].to(self.conv_ring)
        self.state_ring[position % self.state_ring_len] = state.transpose(1, 2).to(self.state_ring)

    def export_state(self, position: int):
        conv = torch.stack(
            [self.conv_ring[(position - 3 + j) % self.conv_ring_len] if position - 3 + j >= 0 else torch.zeros_like(self.conv_ring[0]) for j in range(3)], 1
        )
        return conv, self.state_ring[position % self.state_ring_len].transpose(1, 2).contiguous()
