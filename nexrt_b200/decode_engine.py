"""Batch-1 decode engine: owns the blocks of every layer, the captured whole-step CUDA graphs and
the generate loop.

API of the reference's ``DecodeEngine`` (``nex_n2_5_pro/decode_engine.py:87-399``):
``DecodeEngine(rank, world, dev, cp, ext)``, ``load_prefill``, ``step`` / ``step_cp``, ``capture``,
``generate`` (one-step look-ahead queueing, tokens read from the host mirror), ``status_max``.
What differs: any tensor-parallel width 1/2/4/8; the step carries ``M`` token rows (1 for plain
decode, 4 / 8 for the speculative verifiers and for the engine's own chunked prefill) through the
same kernels; 6 kernel nodes per layer + 3 per step instead of 7-8 + 6, every node launched with
programmatic dependent launch so its weight prefetch overlaps the previous node's tail.
"""

from __future__ import annotations

import os
from typing import Callable, Dict, List, Optional, Sequence

import torch
from .runtime.capture import graph_capture
import torch.distributed as dist

from .attn import FullAttn
from .config import ModelConfig, ShardSpec, active_config
from .ctl_mirror import CtlMirror
from .gdn import Gdn
from .head import MODE_COMMIT, Head
from .moe import Moe
from .ops.lib import check, ptr
from .runtime.context import StepContext
from .runtime.control import CTL_WORDS, Ctl, decode_ctl
from .runtime.rounds import Stops, stop_set

# Context length from which generate() switches to the context-parallel graph.  The reference crosses over at 48K on
# H100 (decode_engine.py:63-66).  On 8 x B200 (groups of four ranks per kv head, full model) the context-parallel arm
# measured 28 us per token slower at 64K (3070 vs 3042 us) and 140 us faster at 256K (3549 vs 3689 us); the straight line
# through the two differences crosses zero at about 96K.
CP_THRESHOLD = int(os.environ.get("NEXRT_CP_THRESHOLD", str(96 * 1024)))
WARMUP_STEPS = 3


class DecodeEngine:
    def __init__(
        self,
        rank: int = 0,
        world: int = 1,
        dev: Optional[torch.device] = None,
        cp: bool = False,
        ext: Optional[Dict] = None,
        *,
        cfg: Optional[ModelConfig] = None,
        group=None,
        max_rows: int = 1,
        cache_len: Optional[int] = None,
        budget_ms: Optional[float] = None,
        shape_tp: Optional[int] = None,
        collective: str = "fused",
    ):
        """``ext`` is the per-rank model dict in kernel layout (``weights.shard_model`` or
        ``weights.random_rank_model``); the reference uses the same argument to alias tensors that
        already live on the device (``decode_engine.py:87-92``)."""
        if ext is None:
            raise ValueError("DecodeEngine needs the per-rank model dict (ext=weights.shard_model(...))")
        self.cfg = cfg or active_config()
        self.rank, self.world = rank, world
        self.dev = dev or torch.device("cuda", torch.cuda.current_device())
        # shape_tp: run alone with the shard shapes of one rank of a shape_tp-wide group (profiling)
        self.spec = ShardSpec(self.cfg, shape_tp or world, rank)
        self.group = group
        self.max_rows = max_rows
        self.cp = bool(cp) and self.spec.cp_size > 1
        self.ctx = StepContext(self.cfg, self.spec, self.dev, group=group, budget_ms=budget_ms, cp=self.cp,
                               comm_world=world, comm_rank=rank, collective=collective)
        state_ring = max(2, max_rows + 1)
        conv_ring = 16
        self.mixers: List = []
        self.moes: List[Moe] = []
        for layer, lw in enumerate(ext["layers"]):
            mw = lw["mixer"]
            if mw["kind"] == "linear":
                self.mixers.append(Gdn(self.ctx, mw, state_ring=state_ring, conv_ring=conv_ring))
            else:
                self.mixers.append(FullAttn(self.ctx, mw, cache_len=cache_len, cp_w=lw.get("mixer_cp") if self.cp else None))
            self.moes.append(Moe(self.ctx, lw["moe"]))
        # the expert gate/up kernel of layer l idles until its router is done: it warms L2 with the projection front of
        # layer l + 1, whose CTAs find no free SM slot early enough to preload their weight rows themselves
        # (same idea as the reference's wait-window prefetch wiring, nex_n2_5_pro/decode_engine.py:154-186)
        # (measured on B200: no gain - the late CTAs are bound by how fast an SM can take 64 KB in, not by where the bytes
        # come from - so the wiring is off unless NEXRT_PREFETCH_FRONT=1)
        if os.environ.get("NEXRT_PREFETCH_FRONT", "0") == "1":
            for layer in range(len(self.mixers) - 1):
                fw = ext["layers"][layer + 1]["mixer"]["front_w"]
                self.moes[layer].prefetch = (fw.data_ptr(), fw.numel() * fw.element_size())
        self.head = Head(self.ctx, ext["head"])
        self.embed = ext["head"]["embed"]
        self.mirror = CtlMirror(self.dev, CTL_WORDS)
        self.graphs: Dict = {}
        self._wide: Dict = {}     # wide prefill paths by (chunk size, activation terms, feature taps)
        self.wide_terms = 0       # activation terms of the wide prefill: 0 = NEXRT_WIDE_TERMS or 3 (the step kernels' exact split); 1 = one e4m3 plane
        self._n_sites: Dict = {}
        # DFlash feature taps: residual rows after the MoE of chosen layers, concatenated per row
        self.tap_layers: Dict[int, int] = {}
        self.taps: Optional[torch.Tensor] = None
        if world > 1:
            dist.barrier(group=group)

    # ---- state --------------------------------------------------------------------------------
    def reset(self, first_token: int = 0, committed_len: int = 0) -> None:
        """Start a new sequence: clear rings and the control block (collective when world > 1)."""
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            dist.barrier(group=self.group)
        for m in self.mixers:
            m.reset()
        c = self.ctx
        c.ctl.zero_()
        c.ctl[Ctl.EOS] = -1
        c.ctl[Ctl.STOP_POS] = -1
        c.ctl[Ctl.COMMITTED_LEN] = committed_len
        c.ctl[Ctl.PENDING] = first_token
        c.ctl[Ctl.IDS] = first_token
        c.channel.reset()
        for wp in self._wide.values():          # the wide prefill path's channel shares the sequence word that just restarted
            if wp.channel is not None:
                wp.channel.buf.tensor.zero_()
        if c.cp_channel is not None:
            c.cp_channel.buf.tensor.zero_()
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            dist.barrier(group=self.group)

    def set_rows(self, ids: Sequence[int]) -> None:
        """Host write of the row ids of the next step (eager use and tests)."""
        t = torch.tensor(list(ids), dtype=torch.int32, device=self.dev)
        self.ctx.ctl[Ctl.IDS : Ctl.IDS + len(ids)] = t

    def set_forced_commit(self, count: int = 0, seed: int = 0, mean10: int = 0) -> None:
        c = self.ctx.ctl
        c[Ctl.FORCED_COMMIT], c[Ctl.FORCED_SEED], c[Ctl.FORCED_MEAN10] = count, seed, mean10

    def read_ctl(self) -> dict:
        return decode_ctl(self.ctx.ctl.tolist())

    @property
    def slot(self):
        """The reference's ``slot = [token, S]`` view of the control block."""
        w = self.ctx.ctl.tolist()
        return [w[Ctl.PENDING], w[Ctl.COMMITTED_LEN]]

    # ---- one step -----------------------------------------------------------------------------
    def step(self, M: int = 1, cp: bool = False, head_mode: int = MODE_COMMIT, end: bool = True, begin: bool = True) -> None:
        """Launch one whole step on the current stream: embed, every layer, head, step end.
        ``begin`` / ``end`` are False when the step is one stage of a longer round (speculative
        modes), whose channel sites are counted across all stages."""
        c = self.ctx
        if begin:
            c.begin_step()
        check(c.lib.nexrt_embed_gather(ptr(self.embed), ptr(c.ctl), ptr(c.x), ptr(c.status), self.cfg.hidden, self.cfg.vocab, M, c.stream()), "embed")
        for layer, (mixer, moe) in enumerate(zip(self.mixers, self.moes)):
            if isinstance(mixer, FullAttn):
                mixer.forward(M, cp=cp)
            else:
                mixer.forward(M)
            moe.forward(M)
            if self.taps is not None and layer in self.tap_layers:
                check(c.lib.nexrt_feature_tap(ptr(c.x), ptr(self.taps), self.cfg.hidden, self.taps.shape[1],
                                              self.tap_layers[layer] * self.cfg.hidden, M, c.stream()), "feature_tap")
        self.head.forward(M, mode=head_mode)
        if end:
            self.step_end()

    def enable_taps(self, layer_ids: Sequence[int]) -> torch.Tensor:
        """Record the residual rows after the MoE of ``layer_ids`` into ``taps [8][n * H]`` on every
        step (reference M8FeatTapKernel, kernels/embed/nex_n2_5_pro_m8_feature_tap_ctypes.cu:45-68)."""
        self.tap_layers = {int(l): i for i, l in enumerate(layer_ids)}
        self.taps = torch.zeros(8, len(self.tap_layers) * self.cfg.hidden, dtype=torch.bfloat16, device=self.dev)
        return self.taps

    def step_cp(self, M: int = 1) -> None:
        self.step(M, cp=True)

    def step_end(self) -> None:
        c = self.ctx
        check(
            c.lib.nexrt_step_end(ptr(c.ctl), ptr(c.seq), c.site, self.mirror.dev_ptr, ptr(self.mirror.gen_dev), CTL_WORDS, c.stream()),
            "step_end",
        )

    def status_max(self) -> int:
        """Largest status word over the ranks (reference decode_engine.py:296-306)."""
        s = self.ctx.ctl[Ctl.STATUS : Ctl.STATUS + 1].clone()
        if self.world > 1:
            dist.all_reduce(s, op=dist.ReduceOp.MAX, group=self.group)
        return int(s.item())

    def logit_gap(self, a: int, b: int, row: int = 0) -> Optional[float]:
        """``|logit[a] - logit[b]|`` of one row of the last step, over the vocabulary shards of all ranks
        (``head.enable_logits()`` must have been called before the step or its capture)."""
        if self.head.logits is None:
            return None
        v, base = self.spec.vocab, self.spec.rank * self.spec.vocab
        vals = torch.full((2,), float("-inf"), dtype=torch.float32, device=self.dev)
        for i, t in enumerate((a, b)):
            if base <= t < base + v:
                vals[i] = self.head.logits[row, t - base]
        if self.world > 1:
            dist.all_reduce(vals, op=dist.ReduceOp.MAX, group=self.group)
        return float((vals[0] - vals[1]).abs().item())

    @property
    def cp_threshold(self) -> int:
        """Context length from which this engine's context-parallel graph is the faster one.  Groups of two ranks never
        win (a rank then walks half the keys for twice the query rows: 4 x B200, 803 vs 790 us per 8 layers at 256K), so
        without an explicit ``NEXRT_CP_THRESHOLD`` the arm stays off for them."""
        if "NEXRT_CP_THRESHOLD" in os.environ or self.spec.cp_size >= 4:
            return CP_THRESHOLD
        return 1 << 30

    # ---- graphs -------------------------------------------------------------------------------
    def capture(self, M: int = 1, cp: bool = False, warmup: int = WARMUP_STEPS):
        """Warm up, then capture one whole step into a CUDA graph (reference
        decode_engine.py:308-324).  The control block is restored afterwards so the capture leaves
        the sequence where it was."""
        key = (M, bool(cp))
        if key in self.graphs:
            return self.graphs[key]
        saved = self._snapshot()
        side = torch.cuda.Stream(device=self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.step(M, cp=cp)
        torch.cuda.current_stream(self.dev).wait_stream(side)
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            dist.barrier(group=self.group)
        g = torch.cuda.CUDAGraph()
        with graph_capture(g, side):
            self.step(M, cp=cp)
        self._restore(saved)
        self.graphs[key] = g
        if self.world > 1:
            dist.barrier(group=self.group)
        return g

    def _snapshot(self):
        torch.cuda.synchronize(self.dev)
        snap = {"ctl": self.ctx.ctl.clone(), "gdn": []}
        C = int(snap["ctl"][Ctl.COMMITTED_LEN])
        for m in self.mixers:
            if isinstance(m, Gdn):
                snap["gdn"].append((m.conv_ring.clone(), m.state_ring[C % m.state_ring_len].clone()))
        return snap

    def _restore(self, snap) -> None:
        torch.cuda.synchronize(self.dev)
        C = int(snap["ctl"][Ctl.COMMITTED_LEN])
        it = iter(snap["gdn"])
        for m in self.mixers:
            if isinstance(m, Gdn):
                conv, st = next(it)
                m.conv_ring.copy_(conv)
                m.state_ring[C % m.state_ring_len].copy_(st)
        self.ctx.ctl.copy_(snap["ctl"])
        self.mirror.resync()
        torch.cuda.synchronize(self.dev)

    # ---- generate -----------------------------------------------------------------------------
    def generate(
        self,
        g_noncp=None,
        g_cp=None,
        max_new: int = 16,
        eos: Stops = None,
        cp_threshold: Optional[int] = None,
        on_tokens: Optional[Callable[[List[int]], None]] = None,
        host_inputs: Optional[torch.Tensor] = None,
    ) -> List[int]:
        """Greedy / sampled decode of up to ``max_new`` tokens by graph replay.

        Step k+1 is queued before step k's token is read from the host mirror, so the GPU never
        idles on the host; EOS is therefore learned one step late and the extra replay is simply
        not reported (reference decode_engine.py:326-399).  ``eos`` is one stop token id or any
        iterable of them.  A token of -1 means a failed step.
        """
        stops = stop_set(eos)
        if cp_threshold is None:
            cp_threshold = self.cp_threshold
        g_noncp = g_noncp or self.capture(1, cp=False)
        if self.cp and g_cp is None:
            g_cp = self.capture(1, cp=True)
        self.mirror.resync()
        S = int(self.ctx.ctl[Ctl.COMMITTED_LEN].item())
        budget = self._kv_budget()
        out: List[int] = []

        def launch(pos: int) -> int:
            if host_inputs is not None:  # per-step upload of the request's sampling words (pinned host memory)
                self.ctx.sampling.copy_(host_inputs, non_blocking=True)
            (g_cp if (g_cp is not None and pos >= cp_threshold) else g_noncp).replay()
            return self.mirror.next_gen()

        pending = [launch(S)]
        queued = 1
        while pending:
            if queued < max_new and S + queued < budget:
                pending.append(launch(S + queued))
                queued += 1
            words = self.mirror.wait(pending.pop(0))
            tok = words[Ctl.EMITTED]
            if tok < 0 or words[Ctl.STATUS] != 0:
                for gen in pending:
                    self.mirror.wait(gen)
                raise RuntimeError(f"decode step failed: status {words[Ctl.STATUS]}")
            out.append(tok)
            if on_tokens:
                on_tokens([tok])
            if tok in stops:
                for gen in pending:
                    self.mirror.wait(gen)
                break
        return out

    def _kv_budget(self) -> int:
        lens = [m.cache_len for m in self.mixers if isinstance(m, FullAttn)]
        return min(lens) if lens else 1 << 30

    # ---- prefill ------------------------------------------------------------------------------
    def prefill(self, ids: Sequence[int], chunk: int = 8, sample: bool = True, resume_from: int = 0,
                on_chunk: Optional[Callable[[int, int], None]] = None, wide: Optional[int] = None) -> int:
        """The engine's own chunked prefill: consume ``ids`` and leave the first generated token
        pending.  This arm runs the multi-row step kernels ``chunk`` rows at a time with a forced full
        commit, so the state it leaves is the decode path's own.  ``resume_from > 0`` keeps the state
        of the first ``resume_from`` tokens (which must be what the engine currently holds) and only
        evaluates the suffix; ``on_chunk(start, end)`` is called after each chunk is queued.  ``wide`` (default: the
        ``NEXRT_WIDE_PREFILL`` environment variable, 0 = off) is the row count of the wide path
        (``prefill_wide.WidePrefill``): whole chunks of that many tokens go through one tcgen05 GEMM per projection,
        the rest of the prompt (at least its last token) through the 8-row steps.  Its activations carry the decode
        kernels' exact three-term split unless ``self.wide_terms`` (or ``NEXRT_WIDE_TERMS``) is 2 or 1 (one e4m3 plane:
        1.65 times the throughput, states equal to the 8-row path's only to FP8 rounding)."""
        if self.max_rows < min(chunk, len(ids)) and len(ids) > 1:
            chunk = self.max_rows
        ids = list(int(t) for t in ids)
        if resume_from:
            have = int(self.ctx.ctl[Ctl.COMMITTED_LEN].item())
            if have != resume_from or resume_from > len(ids):
                raise ValueError(f"cannot resume at {resume_from}: the engine holds {have} tokens")
            if resume_from == len(ids):
                return int(self.ctx.ctl[Ctl.PENDING].item())
        else:
            self.reset(first_token=ids[0])
        pos = resume_from
        wide = int(os.environ.get("NEXRT_WIDE_PREFILL", "0")) if wide is None else int(wide)
        if wide and len(ids) - 1 - pos >= wide:
            wp = self.wide_path(wide)
            if wp is not None:
                n = (len(ids) - 1 - pos) // wide * wide
                wp.run(ids[pos : pos + n], base=pos, on_chunk=on_chunk)
                pos += n
        while pos < len(ids):
            n = min(chunk, len(ids) - pos)
            self.set_rows(ids[pos : pos + n])
            self.set_forced_commit(n)
            g = self.graphs.get((n, False))
            if g is not None:
                g.replay()
            else:
                self.step(n)
            if on_chunk is not None:
                on_chunk(pos, pos + n)
            pos += n
        self.set_forced_commit(0)
        torch.cuda.synchronize(self.dev)
        self.mirror.resync()
        return int(self.ctx.ctl[Ctl.PENDING].item())

    def wide_path(self, rows: int):
        """The wide prefill path for chunks of ``rows`` tokens (built on first use, one per chunk size and per feature-tap
        configuration, because its captured graph contains the taps), or None when the model shapes are outside it."""
        from . import prefill_wide

        if not prefill_wide.supported(self):
            return None
        terms = int(self.wide_terms or os.environ.get("NEXRT_WIDE_TERMS", "3"))
        key = (rows, terms, None if self.taps is None else tuple(sorted(self.tap_layers)))
        wp = self._wide.get(key)
        if wp is None:
            wp = self._wide[key] = prefill_wide.WidePrefill(self, rows, terms=terms)
        return wp

    def load_prefill(self, state: Dict) -> None:
        """Install a saved prefill state ``{L, first_token, layers{idx: {kind, k_cache, v_cache |
        conv_state, recurrent_state}}}`` (reference decode_engine.py:204-233, file format of
        sglang_prefill/extract_state.py:260-281).  Tensors hold this rank's heads."""
        L = int(state["L"])
        self.reset(first_token=int(state["first_token"]), committed_len=L)
        for idx, m in enumerate(self.mixers):
            st = state["layers"][idx]
            if isinstance(m, FullAttn):
                m.load_kv(st["k_cache"].to(self.dev), st["v_cache"].to(self.dev))
            else:
                m.load_state(L, st["conv_state"].to(self.dev), st["recurrent_state"].to(self.dev))
        torch.cuda.synchronize(self.dev)

    def export_state(self) -> Dict:
        """Inverse of :meth:`load_prefill` at the current committed length."""
        w = self.ctx.ctl.tolist()
        L = w[Ctl.COMMITTED_LEN]
        layers = {}
        for idx, m in enumerate(self.mixers):
            if isinstance(m, FullAttn):
                layers[idx] = {"kind": "full", "k_cache": m.k_cache[:, :L].clone(), "v_cache": m.v_cache[:, :L].clone()}
            else:
                conv, st = m.export_state(L)
                layers[idx] = {"kind": "linear", "conv_state": conv.clone(), "recurrent_state": st.clone()}
        return {"rank": self.rank, "tp": self.world, "L": L, "first_token": w[Ctl.PENDING], "layers": layers}


# ---- command line ----------------------------------------------------------------------------------------------
_CLI_MODES = {
    # flag -> (module under nexrt_b200.utils, arguments it adds); everything after the flag is passed through
    "--graph": ("profile_step", ["--graph"]),
    "--profile": ("profile_step", ["--graph", "--leave-one-out"]),
    "--timeline": ("trace_step", []),
    "--scale": ("launch_floor", []),
    "--cp": ("bench_modes", ["--cases", "bs1cp:65536"]),
    "--cp-sweep": ("bench_modes", ["--cases", "bs1:8192,bs1cp:8192,bs1:65536,bs1cp:65536,bs1:131072,bs1cp:131072,bs1:262144,bs1cp:262144"]),
    "--generate": ("bench_modes", ["--cases", "bs1:1024"]),
}


def cli_dispatch(argv):
    """``python -m nexrt_b200.decode_engine MODE [tool arguments]``: the engine's measurement modes under the flag names
    of the reference's ``decode_engine.py`` CLI (eager / ``--graph`` / ``--profile`` / ``--scale`` / ``--cp`` /
    ``--cp-sweep`` / ``--generate``, ``nex_n2_5_pro/decode_engine.py:402-934``).  Each mode is one of the tools under
    ``nexrt_b200/utils``; this returns ``(module name, argument list)`` and ``main`` runs it.  No mode = eager steps."""
    argv = list(argv)
    for flag, (module, extra) in _CLI_MODES.items():
        if flag in argv:
            argv.remove(flag)
            if "--cases" in argv and "--cases" in extra:       # an explicit case list wins over the mode's default
                extra = []
            return module, extra + argv
    return "profile_step", argv


def main(argv=None) -> int:
    import importlib
    import sys

    module, args = cli_dispatch(sys.argv[1:] if argv is None else argv)
    tool = importlib.import_module(f"nexrt_b200.utils.{module}")
    sys.argv = [f"nexrt_b200.utils.{module}"] + args
    out = tool.main()
    return int(out or 0)


if __name__ == "__main__":
    raise SystemExit(main())
