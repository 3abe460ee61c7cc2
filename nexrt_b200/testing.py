"""Small fixtures shared by the tests, the smoke entry point and the examples: a shrunk random
model, its CPU oracle and an engine over it."""

from __future__ import annotations

import functools
from dataclasses import replace

import torch

from .config import ModelConfig, shrunk_config, shrunk_cp_config, shrunk_tp8_config
from .weights import random_checkpoint, shard_model


@functools.lru_cache(maxsize=4)
def shrunk_checkpoint(seed: int = 0, cp: bool = False, kv_heads: int = 0, tp8: bool = False):
    """``kv_heads`` overrides the number of kv heads (1: two ranks already form a context-parallel group); ``tp8`` picks the
    geometry that splits 8 ways."""
    cfg = shrunk_tp8_config() if tp8 else (shrunk_cp_config() if cp else shrunk_config())
    if kv_heads:
        cfg = replace(cfg, name=f"{cfg.name}-kv{kv_heads}", n_kv_heads=kv_heads)
    return cfg, random_checkpoint(cfg, seed)


def make_engine(cfg: ModelConfig, ckpt, rank=0, world=1, device=None, group=None, max_rows=8, cache_len=None, cp=False, budget_ms=None):
    from .decode_engine import DecodeEngine

    device = device or torch.device("cuda", torch.cuda.current_device())
    model = shard_model(ckpt, cfg, world, rank, device, cp=cp)
    return DecodeEngine(rank, world, device, cp=cp, ext=model, cfg=cfg, group=group, max_rows=max_rows,
                        cache_len=cache_len or cfg.cache_len, budget_ms=budget_ms)


def gather_logits(engine, rows: int) -> torch.Tensor:
    """fp32 logits ``[rows, vocab_local]`` of the last step (engine.head.enable_logits() first)."""
    torch.cuda.synchronize()
    return engine.head.logits[:rows].float().cpu()


def attach_silent_peer(engine, budget_ms: float = 50.0) -> None:
    """Turn a single-rank engine's reduce channel into a two-rank channel whose second rank never
    sends: every all-reduce wait then runs out of its (short) budget and latches a status instead of
    completing.  The failure is made on the host (a peer that never joins); the kernels are untouched
    and all their waits stay bounded.  Used by the failure-detection tests."""
    ch = engine.ctx.channel
    if ch.world != 1:
        raise ValueError("attach_silent_peer expects a single-rank engine")
    nbytes = 2 * 2 * ch.slots * 8
    inbox = torch.zeros(nbytes, dtype=torch.uint8, device=engine.dev)
    sink = torch.zeros(nbytes, dtype=torch.uint8, device=engine.dev)     # where packets "to rank 1" land
    s = ch.struct
    engine._silent_peer_buffers = (inbox, sink, (s.local, s.mc, s.peer[0], s.peer[1], s.world, s.rank, s.budget_ns))
    s.local, s.mc = inbox.data_ptr(), None
    s.peer[0], s.peer[1] = inbox.data_ptr(), sink.data_ptr()
    s.world, s.rank = 2, 0
    s.budget_ns = int(budget_ms * 1e6)
    ch.world = 2


def detach_silent_peer(engine) -> None:
    """Undo ``attach_silent_peer``: the channel is the single-rank channel again (the peer "came back")."""
    ch = engine.ctx.channel
    saved = getattr(engine, "_silent_peer_buffers", None)
    if saved is None:
        raise ValueError("no silent peer attached")
    s = ch.struct
    s.local, s.mc, s.peer[0], s.peer[1], s.world, s.rank, s.budget_ns = saved[2]
    ch.world = 1
    torch.cuda.synchronize(engine.dev)
    engine._silent_peer_buffers = None


class RouteAwareCheck:
    """Tolerance policy for comparing a run against the fp32 oracle on RANDOM weights.

    Expert selection is discontinuous: where the oracle's gap between the last selected and the first rejected router
    logit is tiny (``RefModel.margins``, one value per consumed token), two correct evaluations may pick different
    experts, and the outputs then differ by ten percent or more - at that token and, through the caches, mildly at
    every later one.  Tokens with a clear gap are held to ``tol``; a token on a near tie may deviate up to ``loose``, and
    once one of them has actually deviated the clear-gap tokens after it are held to ``4 * tol`` (their caches carry the
    other choice).  A kernel bug shows at the clear-gap tokens too, so it cannot hide behind this."""

    def __init__(self, margins, tol: float = 2e-2, near: float = 0.01, loose: float = 0.3):
        self.margins, self.tol, self.near, self.loose = list(margins), tol, near, loose
        self.flipped = False
        self.strict = 0

    def limit(self, first: int, last: int = None) -> float:
        last = first if last is None else last
        gap = min(self.margins[first : last + 1])
        if gap < self.near:
            return self.loose
        return 4 * self.tol if self.flipped else self.tol

    def check(self, err: float, first: int, last: int = None, what: str = "") -> None:
        limit = self.limit(first, last)
        assert err < limit, (what, first, last, err, limit, min(self.margins[first : (first if last is None else last) + 1]))
        if limit == self.tol:
            self.strict += 1
        elif err >= self.tol:
            self.flipped = True


def oracle_state(ref) -> dict:
    """Per-layer state of a ``RefModel`` in the layout of ``DecodeEngine.export_state`` (whole model)."""
    out = {}
    for idx, st in enumerate(ref.states):
        if st.state is not None:
            out[idx] = {"conv_state": st.conv, "recurrent_state": st.state}
        else:
            out[idx] = {"k_cache": torch.stack(st.k, 1), "v_cache": torch.stack(st.v, 1)}
    return out


def shard_oracle_state(state: dict, cfg: ModelConfig, spec) -> dict:
    """The slice of ``oracle_state`` one tensor-parallel rank holds: its q | k | v conv channels and value heads of every
    gated-delta-net layer, its kv heads of every attention layer (``config.ShardSpec``)."""
    D = cfg.gdn_dim
    out = {}
    for idx, st in state.items():
        if "recurrent_state" in st:
            ql = spec.gdn_qk * D
            q0 = spec.rank * ql
            k0 = cfg.gdn_qk_heads * D + q0
            v0 = 2 * cfg.gdn_qk_heads * D + spec.rank * spec.gdn_v * D
            conv = st["conv_state"]
            out[idx] = {"conv_state": torch.cat([conv[q0 : q0 + ql], conv[k0 : k0 + ql], conv[v0 : v0 + spec.gdn_v * D]]),
                        "recurrent_state": st["recurrent_state"][spec.rank * spec.gdn_v : (spec.rank + 1) * spec.gdn_v]}
        else:
            sl = slice(spec.kv_head0, spec.kv_head0 + spec.kv_heads)
            out[idx] = {"k_cache": st["k_cache"][sl], "v_cache": st["v_cache"][sl]}
    return out
