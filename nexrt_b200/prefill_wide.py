"""Wide prefill: prompt chunks of 16..128 tokens per pass instead of the 8-row steps of ``DecodeEngine.prefill``.

The reference hands prefill to SGLang (``nex_n2_5_pro/sglang_prefill/bridge.py:310-398``, 4096-token extends); this
engine prefills through its own kernels, and at 8 rows per step every weight of the model is streamed once per 8
tokens.  Here a chunk of ``T`` rows goes through each layer in one pass:

* every projection (GDN / attention fronts, out-projections, router, expert gate/up and down) is one tcgen05 GEMM
  over all ``T`` rows (``csrc/tc_gemm.cu``): e4m3 activations with one scale per row and 128 columns, the
  checkpoint's block-scaled FP8 weights, fp32 accumulation - every weight byte is read once per chunk;
* the experts run **dense**: the gate/up GEMM multiplies the chunk by all ``E + 1`` experts (with 64 rows x 10
  routes nearly every expert is used anyway, and the FP8 tensor cores make the extra columns cheaper than a
  gather), a small kernel turns the routed ``(row, expert)`` pairs into quantised ``h`` and leaves a zero scale
  everywhere else, and the down GEMM walks ``K = (E + 1) * I`` split over CTAs;
* the GDN layer's conv ring, gates and delta rule run over the whole chunk in two kernels (``csrc/prefill.cu``: the
  step kernels' arithmetic, the recurrent state kept in registers along the chunk);
* causal attention reuses the multi-row decode kernel eight rows at a time: the chunk's q / gate / k rows are scattered
  and its K rows (norm + RoPE) published to the cache first, so the sub-steps do not depend on each other and run
  side by side on their own streams; sub-step ``j`` reads its base position from entry ``j`` of a control-block table,
  which makes the chunk position-independent on the host: it is captured once into a CUDA graph and replayed;
* on a tensor-parallel group the residual add also all-reduces the chunk's partial sums inside the kernel (vector
  stores through the multicast alias or to each peer, one tagged flag word per CTA), so the graph holds the whole
  chunk on every rank.

The state it leaves (conv / state rings, KV cache, committed length) is the decode path's own, so decode - or the
8-row prefill of the prompt's tail - continues from it.

Activation precision (``terms``).  With one term the activations of every FP8 product are one e4m3 plane (a scale per row
and 128 columns), so hidden states agree with the 8-row path to FP8 rounding only; the same holds between the reference's
SGLang prefill and its decode kernels.  With two or three terms the quantisers write the step kernels' split
(``x = s (t1 + t2 / 16 + t3 / 256)``) as further row blocks of the activation matrix: the GEMM runs over ``terms * T``
token rows against the same weight tiles (which it still streams from memory once), and whoever consumes its output adds
the row blocks like K-split partial sums.  Three terms reproduce the decode arithmetic to 2^-12 per activation.
"""

from __future__ import annotations

import weakref
from typing import List, Sequence

import torch
from .runtime.capture import graph_capture

from .attn import FullAttn
from .ops.lib import check, ptr
from .ops.tc_gemm import bf16_gemm_split, fp8_gemm, fp8_gemm_split
from .quant import FP8
from .runtime.control import CTL_WORDS, Ctl

SUB = 8   # rows per sub-step of the sequential kernels


def supported(eng) -> bool:
    """Shapes the wide path covers: everything the tcgen05 GEMMs tile (128-row weight tiles, 128-wide K blocks)."""
    cfg, spec = eng.cfg, eng.spec
    return (
        eng.max_rows >= SUB
        and cfg.hidden % 128 == 0 and cfg.hidden <= 8192 and spec.inter % 128 == 0
        and spec.gdn_front_rows % 128 == 0 and spec.attn_front_rows % 128 == 0
        and spec.gdn_local % 128 == 0 and spec.gdn_local <= 8192 and spec.attn_local % 128 == 0 and spec.attn_local <= 8192
        and cfg.hidden // 64 <= 64 and cfg.gdn_dim == 128
    )


def down_split(k_blocks: int, tiles: int, n_cta: int, max_blocks: int = 64, max_split: int = 16) -> int:
    """Number of K ranges of the expert down product: every CTA walks at most ``max_blocks`` K blocks, the grid
    (``tiles`` output tiles x ranges) has about two CTAs per SM, and every range is non-empty (the split is a fixed
    point of ``ceil(k_blocks / ceil(k_blocks / split))``, which is what the kernel launcher derives its ranges from)."""
    ks = max((k_blocks + max_blocks - 1) // max_blocks, min(k_blocks, max_split, max(1, 2 * n_cta // max(tiles, 1))))
    while True:
        per = (k_blocks + ks - 1) // ks
        eff = (k_blocks + per - 1) // per
        if eff == ks:
            return ks
        ks = eff


class WidePrefill:
    def __init__(self, eng, chunk: int = 64, graph: bool = True, terms: int = 3):
        if chunk % SUB or chunk < 2 * SUB or chunk > 128:
            raise ValueError("chunk must be a multiple of 8 between 16 and 128")
        if terms not in (1, 2, 3):
            raise ValueError("terms must be 1, 2 or 3")
        if not supported(eng):
            raise ValueError("model shapes outside the wide prefill path")
        self.eng, self.T, self.use_graph = weakref.proxy(eng), chunk, graph     # the engine owns this object: no reference cycle
        c, cfg, spec, dev = eng.ctx, eng.cfg, eng.spec, eng.dev
        T, H = chunk, cfg.hidden
        P = self.P = terms            # e4m3 planes per activation = row blocks of every FP8 product's token side
        f32, bf, i32 = torch.float32, torch.bfloat16, torch.int32
        z = lambda *shape, dtype=f32: torch.zeros(*shape, dtype=dtype, device=dev)
        self.n_sub = T // SUB
        self.ids = z(T, dtype=i32)
        self.x = z(T, H, dtype=bf)
        self.xq, self.sx = torch.zeros(P * T, H, dtype=FP8, device=dev), z(P * T, H // 128)
        self.xn = z(T, H)
        self.planes = z(T, 2 * H, dtype=bf)
        kb = H // 128
        self.front_ksplit = next(k for k in (4, 2, 1) if kb % k == 0)     # K split of the GDN front projection (few row tiles)
        self.pre = z(P * T * max(self.front_ksplit * spec.gdn_front_rows, spec.attn_front_rows))
        self.pre_sum = z(T, spec.attn_front_rows) if P > 1 else None
        self.ctl_tab = z(self.n_sub, CTL_WORDS, dtype=i32)
        self.gdn_qkv, self.gdn_z = z(T, spec.gdn_qkv_rows), z(T, spec.gdn_local)
        self.gdn_beta, self.gdn_g, self.gdn_out = z(T, spec.gdn_v), z(T, spec.gdn_v), z(T, spec.gdn_local)
        self.gate, self.attn_out = z(T, spec.q_heads, cfg.head_dim), z(T, spec.attn_local)
        self.q_raw, self.k_raw = z(T, spec.q_heads, cfg.head_dim), z(T, spec.kv_heads, cfg.head_dim)
        # the attention sub-steps of a chunk run side by side: one split-KV workspace, ticket and stream per sub-step
        self.ws_acc = z(self.n_sub, *c.ws_acc.shape)
        self.ws_ml = z(self.n_sub, *c.ws_ml.shape)
        self.attn_ticket = z(self.n_sub, spec.kv_heads, dtype=i32)
        self.side = [torch.cuda.Stream(dev) for _ in range(self.n_sub)]
        kmax = max(spec.gdn_local, spec.attn_local)
        self.oq, self.os = torch.zeros(P * T * kmax, dtype=FP8, device=dev), z(P * T * (kmax // 128))
        self.S, self.n_total = cfg.top_k + 1, cfg.n_experts + 1
        self.rows_pad = eng.moes[0].rows_pad
        kb64 = H // 64
        self.router_ksplit = next(k for k in (8, 4, 2, 1) if kb64 % k == 0)
        self.logits = z(2 * self.router_ksplit, T, self.rows_pad)
        self.moe_logits, self.moe_ids, self.moe_wts = z(T, cfg.n_experts + 1), z(T, self.S, dtype=i32), z(T, self.S)
        I = spec.inter
        self.used = z(self.n_total, dtype=i32)
        # K split of the gate/up product: 1 (two half-length CTAs per tile fill the last wave better but write and re-read a
        # second 34 MB plane: measured 4 % slower per chunk at 64 rows)
        self.up_ksplit = 1
        self.gu = z(self.up_ksplit, P * T, self.n_total * 2 * I)
        self.hq, self.hs = torch.zeros(P * T, self.n_total * I, dtype=FP8, device=dev), z(P * T, self.n_total * I // 128)
        # K split of the expert down product: at most 64 K blocks per CTA, and about two CTAs per SM over the grid
        self.down_ksplit = down_split(self.n_total * I // 128, (H // 128) * ((P * T + 63) // 64), c.n_cta)
        self.y = z(max(self.down_ksplit, 1), P * T, H)
        # tensor parallel: the chunk's partial sums are all-reduced inside the residual kernel over a symmetric inbox of its
        # own (8 bytes per value of the chunk and half: data vectors, then one flag word per CTA); it shares the engine's
        # sequence word and status, so its tags never collide with the decode steps' and a failure stops both
        self.channel = None
        if eng.world > 1:
            from .parallel.channel import LLChannel

            self.channel = LLChannel(dev, eng.world, eng.rank, T * H, group=eng.group, seq=c.seq, status=c.status)
            self.channel.struct.budget_ns = c.channel.struct.budget_ns
        # feature taps (DFlash): the residual rows after the MoE of the tapped layers, concatenated per row like the
        # engine's 8-row tap buffer
        self.taps = None if eng.taps is None else torch.zeros(T, eng.taps.shape[1], dtype=bf, device=dev)
        self.tap_layers = dict(eng.tap_layers)
        self.site = 0
        self.graph = None

    # ---- one chunk ---------------------------------------------------------------------------------------------
    def _finish(self, ksplit: int) -> None:
        """x += (all-reduced) sum of the projection's K-split planes, each of which holds one row block per activation term."""
        c, lib, st = self.eng.ctx, self.eng.ctx.lib, self.eng.ctx.stream()
        n = self.T * self.eng.cfg.hidden
        ksplit *= self.P
        if self.channel is None:
            check(lib.nexrt_planes_residual(ptr(self.x), ptr(self.y), None, n, ksplit, st), "planes_residual")
            return
        check(lib.nexrt_planes_allreduce_residual(ptr(self.x), ptr(self.y), n, ksplit, self.channel.ref, self.site, st), "planes_allreduce_residual")
        self.site += 1

    def _gdn(self, m) -> None:
        eng, T = self.eng, self.T
        c, lib, cfg, spec = eng.ctx, eng.ctx.lib, eng.cfg, eng.spec
        st, w, H = c.stream(), m.w, cfg.hidden
        R, C, nv, K = spec.gdn_front_rows, spec.gdn_qkv_rows, spec.gdn_v, spec.gdn_local
        P = self.P
        check(lib.nexrt_norm_rows(ptr(self.x), ptr(w["in_ln"]), ptr(self.xq), ptr(self.sx), ptr(self.xn), None, H, T, cfg.rms_eps, P, st), "norm_rows")
        ks = self.front_ksplit
        pre = self.pre[: ks * P * T * R]         # [ks][P][T][R]: ks * P planes of T rows for the chunk kernel
        fp8_gemm_split(w["front_w"], w["front_s"], self.xq, self.sx, pre, ksplit=ks, status=c.status)
        # conv ring + gates and the delta rule for all T rows: two kernels, the state carried in registers along the chunk
        check(
            lib.nexrt_gdn_chunk(ptr(pre), ptr(self.xn), ptr(w["ba_w_pad"]), ptr(w["conv_w"]), ptr(w["a_log"]), ptr(w["dt_bias"]), ptr(self.ctl_tab[0]),
                                ptr(m.conv_ring), ptr(self.gdn_qkv), ptr(self.gdn_z), ptr(self.gdn_beta), ptr(self.gdn_g), ptr(m.state_ring), ptr(self.gdn_out),
                                H, R, C, nv, spec.gdn_qk, T, m.conv_ring_len, m.state_ring_len, ks * P, st),
            "gdn_chunk",
        )
        oq, os_ = self.oq[: P * T * K].view(P * T, K), self.os[: P * T * (K // 128)].view(P * T, K // 128)
        check(lib.nexrt_gdn_gate_quant(ptr(self.gdn_out), ptr(self.gdn_z), ptr(w["gnorm_w"]), ptr(oq), ptr(os_), K, T, cfg.rms_eps, P, st), "gdn_gate_quant")
        fp8_gemm(w["out_w"], w["out_s"], oq, os_, out=self.y[0], status=c.status)
        self._finish(1)

    def _attn(self, m: FullAttn) -> None:
        eng, T = self.eng, self.T
        c, lib, cfg, spec = eng.ctx, eng.ctx.lib, eng.cfg, eng.spec
        st, w, H, hd = c.stream(), m.w, cfg.hidden, cfg.head_dim
        nq, kvh, K = spec.q_heads, spec.kv_heads, spec.attn_local
        R = spec.attn_front_rows
        P = self.P
        check(lib.nexrt_norm_rows(ptr(self.x), ptr(w["in_ln"]), ptr(self.xq), ptr(self.sx), None, None, H, T, cfg.rms_eps, P, st), "norm_rows")
        pre = self.pre[: P * T * R].view(P * T, R)
        fp8_gemm(w["front_w"], w["front_s"], self.xq, self.sx, out=pre, status=c.status)
        if P > 1:                               # the scatter kernels below read one plane: add the terms' row blocks first
            check(lib.nexrt_planes_residual(None, ptr(pre), ptr(self.pre_sum), T * R, P, st), "planes_sum")
            pre = self.pre_sum
        rope = c.rope_table(m.cache_len)
        base = self.ctl_tab[0]
        # q / gate / k rows to scratch and v rows to the cache for the whole chunk, then the chunk's k rows (norm + RoPE) to
        # the cache: after that the 8-row attention sub-steps do not depend on each other and run side by side
        check(lib.nexrt_attn_front_tail(ptr(pre), ptr(base), ptr(self.q_raw), ptr(self.gate), ptr(self.k_raw), ptr(m.v_cache), hd, nq, nq, kvh, T,
                                        m.cache_len, 1, st), "attn_front_tail")
        check(lib.nexrt_kv_publish(ptr(pre), R, 2 * nq * hd, (2 * nq + kvh) * hd, ptr(w["kn"]), ptr(rope), ptr(base), ptr(m.k_cache), ptr(m.v_cache), hd, kvh, T,
                                   m.cache_len, cfg.rotary_dim, cfg.rms_eps, 0, st), "kv_publish")
        cur = torch.cuda.current_stream(eng.dev)
        for j in range(self.n_sub):
            r = slice(j * SUB, (j + 1) * SUB)
            side = self.side[j]
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                check(
                    lib.nexrt_attn_decode(ptr(self.q_raw[r]), ptr(self.gate[r]), ptr(self.k_raw[r]), ptr(w["qn"]), ptr(w["kn"]), ptr(c.inv_freq), ptr(rope),
                                          ptr(self.ctl_tab[j]), ptr(m.k_cache), ptr(m.v_cache), ptr(self.ws_acc[j]), ptr(self.ws_ml[j]), ptr(self.attn_ticket[j]),
                                          ptr(self.attn_out[r]), hd, nq, nq, kvh, SUB, m.cache_len, cfg.rotary_dim, c.n_splits, cfg.rms_eps, 4, 0, 0, 0, 1, 0,
                                          None, 0, c.stream()),
                    "attn_decode",
                )
        for j in range(self.n_sub):
            cur.wait_stream(self.side[j])
        oq, os_ = self.oq[: P * T * K].view(P * T, K), self.os[: P * T * (K // 128)].view(P * T, K // 128)
        check(lib.nexrt_act_quant(ptr(self.attn_out), 1, K, None, cfg.rms_eps, ptr(oq), ptr(os_), T, K, P, st), "act_quant")
        fp8_gemm(w["out_w"], w["out_s"], oq, os_, out=self.y[0], status=c.status)
        self._finish(1)

    def _moe(self, moe) -> None:
        eng, T = self.eng, self.T
        c, lib, cfg, spec = eng.ctx, eng.ctx.lib, eng.cfg, eng.spec
        st, w, H, I, S, n_total = c.stream(), moe.w, cfg.hidden, spec.inter, self.S, self.n_total
        P = self.P
        check(lib.nexrt_norm_rows(ptr(self.x), ptr(w["post_ln"]), ptr(self.xq), ptr(self.sx), None, ptr(self.planes), H, T, cfg.rms_eps, P, st), "norm_rows")
        # router: bf16 weights, activations as hi + lo bf16 planes, each product split over K; the top-k kernel adds the
        # 2 * ksplit partial planes in a fixed order (one CTA per eight rows)
        ks = self.router_ksplit
        bf16_gemm_split(w["router_w_pad"], self.planes[:, :H], self.logits[:ks], ks, status=c.status)
        bf16_gemm_split(w["router_w_pad"], self.planes[:, H:], self.logits[ks:], ks, status=c.status)
        check(lib.nexrt_moe_router_topk(ptr(self.logits), 2 * ks, self.rows_pad, ptr(self.moe_logits), ptr(self.moe_ids), ptr(self.moe_wts),
                                        cfg.n_experts, cfg.top_k, T, st), "moe_router_topk")
        # experts, dense: gate/up of every expert for every row, activation of the routed pairs, down over all experts
        # (experts no row of the chunk routes to are skipped: their weights are not read)
        check(lib.nexrt_moe_mark_used(ptr(self.moe_ids), ptr(self.used), T * S, n_total, st), "moe_mark_used")
        fp8_gemm_split(w["w13"].view(n_total * 2 * I, H), w["w13_s"].view(-1, H // 128), self.xq, self.sx, self.gu, ksplit=self.up_ksplit, used=self.used, used_rows=2 * I,
                       status=c.status)
        self.hq.view(torch.uint8).zero_()
        self.hs.zero_()
        check(lib.nexrt_moe_dense_act(ptr(self.gu), ptr(self.moe_ids), ptr(self.moe_wts), ptr(self.hq), ptr(self.hs), I, S, T, n_total, self.up_ksplit * P, P, st),
              "moe_dense_act")
        fp8_gemm_split(w["w2"].view(n_total * H, I), w["w2_s"], self.hq, self.hs, self.y, ksplit=self.down_ksplit, group_k=I, group_rows=H, used=self.used, status=c.status)
        self._finish(self.down_ksplit)

    def _chunk(self) -> None:
        """All layers over the rows named by ``self.ids`` at the engine's committed length, which then advances by T."""
        eng = self.eng
        c, lib, st = eng.ctx, eng.ctx.lib, eng.ctx.stream()
        self.site = 0
        check(lib.nexrt_prefill_ctl(ptr(c.ctl), ptr(self.ctl_tab), self.n_sub, SUB, st), "prefill_ctl")
        check(lib.nexrt_prefill_embed(ptr(eng.embed), ptr(self.ids), ptr(self.x), ptr(c.status), eng.cfg.hidden, eng.cfg.vocab, self.T, st), "prefill_embed")
        for layer, (mixer, moe) in enumerate(zip(eng.mixers, eng.moes)):
            if isinstance(mixer, FullAttn):
                self._attn(mixer)
            else:
                self._gdn(mixer)
            self._moe(moe)
            if self.taps is not None and layer in self.tap_layers:
                check(lib.nexrt_feature_tap(ptr(self.x), ptr(self.taps), eng.cfg.hidden, self.taps.shape[1], self.tap_layers[layer] * eng.cfg.hidden, self.T, st),
                      "feature_tap")
        check(lib.nexrt_prefill_advance(ptr(c.ctl), self.T, ptr(c.seq), self.site, st), "prefill_advance")

    def run(self, ids: Sequence[int], base: int = 0, on_chunk=None, after_chunk=None) -> None:
        """Consume ``len(ids)`` (a multiple of the chunk size) prompt tokens starting at the engine's committed length
        (``base``, only used to report progress through ``on_chunk(start, end)``).  ``after_chunk(start, x)`` is called once
        a chunk is queued, with ``x [T, H]`` the residual rows after the last layer (speculative-decoding drafts that follow
        the target's hidden states queue their own work on them before the next chunk overwrites the buffer)."""
        if len(ids) % self.T:
            raise ValueError("the wide path takes whole chunks")
        dev = self.eng.dev
        for pos in range(0, len(ids), self.T):
            self.ids.copy_(torch.tensor(list(ids[pos : pos + self.T]), dtype=torch.int32), non_blocking=False)
            if on_chunk is not None:
                on_chunk(base + pos, base + pos + self.T)
            if not self.use_graph:
                self._chunk()
                if after_chunk is not None:
                    after_chunk(base + pos, self.x)
                continue
            if self.graph is None:
                # one eager pass (lazy initialisation in the launchers must not happen under capture), whose state
                # changes are undone before the captured pass is replayed for the same rows
                snap = self._snapshot()
                self._chunk()
                torch.cuda.synchronize(dev)
                self._restore(snap)
                g = torch.cuda.CUDAGraph()
                s = torch.cuda.Stream(dev)
                s.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(s):
                    with graph_capture(g, s):
                        self._chunk()
                torch.cuda.current_stream(dev).wait_stream(s)
                torch.cuda.synchronize(dev)
                self._restore(snap)
                self.graph = g
            self.graph.replay()
            if after_chunk is not None:
                after_chunk(base + pos, self.x)
        torch.cuda.synchronize(dev)

    # the eager warm-up pass and the capture itself touch the rings, the caches and the committed length
    def _snapshot(self) -> List:
        eng = self.eng
        snap: List = [eng.ctx.ctl.clone()]
        C0 = int(eng.ctx.ctl[Ctl.COMMITTED_LEN].item())
        for m in eng.mixers:
            if isinstance(m, FullAttn):
                snap.append((m.k_cache[:, C0 : C0 + self.T].clone(), m.v_cache[:, C0 : C0 + self.T].clone(), C0))
            else:
                snap.append((m.conv_ring.clone(), m.state_ring.clone()))
        return snap

    def _restore(self, snap: List) -> None:
        eng = self.eng
        eng.ctx.ctl.copy_(snap[0])
        for m, s in zip(eng.mixers, snap[1:]):
            if isinstance(m, FullAttn):
                k, v, C0 = s
                m.k_cache[:, C0 : C0 + self.T] = k
                m.v_cache[:, C0 : C0 + self.T] = v
            else:
                m.conv_ring.copy_(s[0])
                m.state_ring.copy_(s[1])
