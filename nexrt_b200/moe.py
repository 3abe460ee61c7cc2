"""Mixture-of-experts block: router + top-k, expert gate/up, expert down fused with the all-reduce.

Counterpart of the reference's ``Moe`` (``nex_n2_5_pro/moe.py:220-426``): 512 routed experts,
top-10 with renormalised softmax weights, one shared expert gated by ``sigmoid(gate . x)``,
intermediate-parallel sharding (every rank holds all experts, ``inter / tp`` columns of each).
Three launches instead of four (router GEMV and top-k are one kernel) and the raw weight mode
only: the post-attention RMSNorm multiplier is applied to the activation in the kernels, so
checkpoint tensors are used as stored (the reference's folded mode re-quantises every expert,
``moe.py:127-171``).
"""

from __future__ import annotations

import os

import torch

from .ops.lib import check, ptr
from .runtime.context import StepContext


class Moe:
    def __init__(self, ctx: StepContext, w: dict):
        self.ctx, self.w = ctx, w
        rw = w["router_w"]
        self.rows_pad = (rw.shape[0] + 15) // 16 * 16   # the reference pads the router to 528 rows too (moe.py:127-171)
        if "router_w_pad" not in w:
            pad = torch.zeros(self.rows_pad, rw.shape[1], dtype=rw.dtype, device=rw.device)
            pad[: rw.shape[0]] = rw
            w["router_w_pad"] = pad
        # rows from which the experts run on the tcgen05 kernels (NEXRT_TC_MOE_ROWS=0 switches them off)
        self.tc_rows = int(os.environ.get("NEXRT_TC_MOE_ROWS", "2")) or 1 << 30
        self.tc_router_rows = int(os.environ.get("NEXRT_TC_ROUTER_ROWS", "8")) or 1 << 30   # below 8 rows the fused router kernel is as fast
        cfg, spec = ctx.cfg, ctx.spec
        self.tc_ok = cfg.hidden % 128 == 0 and cfg.hidden <= 4096 and spec.inter % 128 == 0
        # the fused router takes its tensor-core form (the one that can also write the planes) under these conditions
        self.router_mma = (int(os.environ.get("NEXRT_GEMV_MODE", "255")) & 16) != 0 and cfg.hidden % 1024 == 0 and cfg.hidden <= 4096
        self._planes_ready = False
        # routed pair (router stops at partial logits, the gate/up kernel selects): NEXRT_MOE_ROUTED=0 goes back to the
        # router with the one-CTA top-k tail
        gm = int(os.environ.get("NEXRT_GEMV_MODE", "255"))
        self.routed_ok = (os.environ.get("NEXRT_MOE_ROUTED", "1") != "0" and (gm & 4) != 0 and (gm & 16) != 0 and cfg.hidden % 1024 == 0
                          and cfg.hidden <= 4096 and spec.inter % 128 == 0)
        self.prefetch = None          # (address, bytes) of a later kernel's constant weights, set by the engine
        self.prefetch_w2 = os.environ.get("NEXRT_PREFETCH_W2", "0") == "1"      # measured: no gain on B200, off by default

    def forward(self, M: int = 1) -> None:
        c, w, lib = self.ctx, self.w, self.ctx.lib
        cfg, spec, st = c.cfg, c.spec, c.stream()
        S = cfg.top_k + 1
        wide = M >= self.tc_router_rows and self.tc_ok and cfg.hidden % (64 * c.router_ksplit) == 0
        tc_experts = M >= self.tc_rows and self.tc_ok
        # the routers of a step whose experts run on tcgen05 also leave the experts' activation planes
        self._planes_ready = tc_experts and (wide or self.router_mma)
        planes = ptr(c.moe_planes1) if self._planes_ready else None
        if wide:
            # multi-row steps: router logits of all rows in one tcgen05 GEMM (bf16 weights, hi + lo activation planes,
            # K split over CTAs), then one small kernel adds the partial planes and selects the experts
            check(
                lib.nexrt_tc_router_logits(ptr(c.x), ptr(w["post_ln"]), ptr(w["router_w_pad"]), ptr(c.router_planes), ptr(c.router_partial), ptr(c.zero_ids),
                                           cfg.n_experts + 1, self.rows_pad, cfg.hidden, M, c.router_ksplit, cfg.rms_eps, planes, ptr(c.status), st),
                "tc_router_logits",
            )
            check(lib.nexrt_moe_router_topk(ptr(c.router_partial), c.router_ksplit, self.rows_pad, ptr(c.moe_logits), ptr(c.moe_ids), ptr(c.moe_wts),
                                            cfg.n_experts, cfg.top_k, M, st), "moe_router_topk")
        elif not tc_experts and self.routed_ok:
            self._routed(M)
            return
        elif self.routed_ok and self.router_mma:
            # a few rows with the experts on tcgen05: the router stops at its partial logits (no ticket, no one-CTA tail)
            # and a one-CTA node adds them and selects - two short nodes instead of one long one
            check(lib.nexrt_moe_router_partial(ptr(c.x), ptr(w["post_ln"]), ptr(w["router_w_pad"]), ptr(c.moe_partial), self.rows_pad, cfg.hidden,
                                               cfg.n_experts, cfg.top_k, M, cfg.rms_eps, planes, st), "moe_router_partial")
            check(lib.nexrt_moe_router_topk(ptr(c.moe_partial), lib.nexrt_moe_router_partial_split(), self.rows_pad, ptr(c.moe_logits),
                                            ptr(c.moe_ids), ptr(c.moe_wts), cfg.n_experts, cfg.top_k, M, st), "moe_router_topk")
        else:
            self._router_fused(M, planes)
        self._experts(M)

    def _routed(self, M: int) -> None:
        """One-row form (and any step whose experts stay on the ``mma.sync`` kernels): the router stops at its partial
        logits, the gate/up kernel selects the experts itself and warms L2 for the kernels behind it."""
        c, w, lib = self.ctx, self.w, self.ctx.lib
        cfg, spec, st = c.cfg, c.spec, c.stream()
        check(lib.nexrt_moe_router_partial(ptr(c.x), ptr(w["post_ln"]), ptr(w["router_w_pad"]), ptr(c.moe_partial), self.rows_pad, cfg.hidden,
                                           cfg.n_experts, cfg.top_k, M, cfg.rms_eps, None, st), "moe_router_partial")
        pf, pf_bytes = self.prefetch if (self.prefetch is not None and M == 1) else (None, 0)
        check(lib.nexrt_moe_l1_routed(ptr(c.x), ptr(w["post_ln"]), ptr(w["w13"]), ptr(w["w13_s"]), ptr(c.moe_partial), self.rows_pad, ptr(c.moe_ids),
                                      ptr(c.moe_wts), ptr(c.moe_logits), ptr(c.moe_gu), ptr(w["w2"]) if self.prefetch_w2 else None, pf, pf_bytes,
                                      cfg.hidden, spec.inter, cfg.n_experts, cfg.top_k, M, cfg.rms_eps, st), "moe_l1_routed")
        check(
            lib.nexrt_moe_l2_allreduce(
                ptr(c.moe_gu), ptr(c.moe_ids), ptr(c.moe_wts), ptr(w["w2"]), ptr(w["w2_s"]), ptr(c.x), cfg.hidden, spec.inter, cfg.top_k + 1, M,
                c.ar_channel.ref, c.next_site(), c.n_cta, st,
            ),
            "moe_l2_allreduce",
        )
        c.after_allreduce(M)

    def _router_fused(self, M: int, planes=None) -> None:
        c, w, lib = self.ctx, self.w, self.ctx.lib
        cfg, spec, st = c.cfg, c.spec, c.stream()
        check(
            lib.nexrt_moe_router(
                ptr(c.x), ptr(w["post_ln"]), ptr(w["router_w_pad"]), ptr(c.moe_logits), ptr(c.moe_ids), ptr(c.moe_wts), ptr(c.moe_ticket),
                ptr(c.moe_partial), self.rows_pad, cfg.hidden, cfg.n_experts, cfg.top_k, M, cfg.rms_eps, c.n_cta, planes, st,
            ),
            "moe_router",
        )

    def _experts(self, M: int) -> None:
        c, w, lib = self.ctx, self.w, self.ctx.lib
        cfg, spec, st = c.cfg, c.spec, c.stream()
        S = cfg.top_k + 1
        if M >= self.tc_rows and self.tc_ok:
            # multi-row steps: experts on the tcgen05 tensor cores, each distinct expert streamed once, the
            # tensor-parallel all-reduce fused into the down projection's epilogue (csrc/tc_moe.cu)
            n_total = cfg.n_experts + 1
            # K split of the gate/up product: two CTAs per expert tile while they all fit one wave (two per SM)
            tiles = M * S * (2 * spec.inter // 128)
            ks = c.moe_ksplit if tiles * c.moe_ksplit <= 2 * c.n_cta else 1
            check(
                lib.nexrt_tc_moe_l1(ptr(c.x), ptr(w["post_ln"]), ptr(w["w13"]), ptr(w["w13_s"]), ptr(c.moe_ids), ptr(c.moe_gu_tc), ptr(c.moe_planes1),
                                    cfg.hidden, spec.inter, S, M, n_total, ks, cfg.rms_eps, int(self._planes_ready), ptr(c.status), st),
                "tc_moe_l1",
            )
            check(
                lib.nexrt_tc_moe_l2_allreduce(ptr(c.moe_gu_tc), ptr(c.moe_ids), ptr(c.moe_wts), ptr(w["w2"]), ptr(w["w2_s"]), ptr(c.x), ptr(c.moe_planes2),
                                              ptr(c.moe_descale), cfg.hidden, spec.inter, S, M, n_total, ks, c.channel.ref, c.next_site(),
                                              ptr(c.status), st),
                "tc_moe_l2_allreduce",
            )
            return
        check(
            lib.nexrt_moe_l1(
                ptr(c.x), ptr(w["post_ln"]), ptr(w["w13"]), ptr(w["w13_s"]), ptr(c.moe_ids), ptr(c.moe_gu), cfg.hidden, spec.inter, S, M,
                cfg.rms_eps, cfg.n_experts, c.n_cta, st,
            ),
            "moe_l1",
        )
        check(
            lib.nexrt_moe_l2_allreduce(
                ptr(c.moe_gu), ptr(c.moe_ids), ptr(c.moe_wts), ptr(w["w2"]), ptr(w["w2_s"]), ptr(c.x), cfg.hidden, spec.inter, S, M,
                c.ar_channel.ref, c.next_site(), c.n_cta, st,
            ),
            "moe_l2_allreduce",
        )
        c.after_allreduce(M)
