"""Capture and serve loop of DFlash speculative decoding (reference ``nex_n2_5_pro/dflash/serve.py``:
``capture_request`` ``:29-45``, ``generate_dflash`` ``:48-121``)."""

from __future__ import annotations

from typing import Callable, List, Optional

import torch
from ..runtime.capture import graph_capture
import torch.distributed as dist

from ..runtime.control import Ctl
from .block import M8, DFlashBlock


def capture_request(block: DFlashBlock, cp: bool = False, warmup: int = 3):
    """Capture one round.  The graph does not depend on the request (base positions are read from
    device memory), so it is captured once and reused; the name is kept for API compatibility."""
    eng = block.eng
    key = ("dflash", bool(cp))
    if key in eng.graphs:
        return eng.graphs[key]
    saved = eng._snapshot()
    side = torch.cuda.Stream(device=eng.dev)
    side.wait_stream(torch.cuda.current_stream(eng.dev))
    with torch.cuda.stream(side):
        for _ in range(warmup):
            block.round(cp=cp)
    torch.cuda.current_stream(eng.dev).wait_stream(side)
    torch.cuda.synchronize(eng.dev)
    if eng.world > 1:
        dist.barrier(group=eng.group)
    g = torch.cuda.CUDAGraph()
    with graph_capture(g, side):
        block.round(cp=cp)
    eng._restore(saved)
    eng.graphs[key] = g
    if eng.world > 1:
        dist.barrier(group=eng.group)
    return g


def generate_dflash(block: DFlashBlock, graph=None, max_new: int = 16, eos: Optional[int] = None,
                    on_tokens: Optional[Callable[[List[int]], None]] = None, stats: Optional[dict] = None) -> List[int]:
    eng = block.eng
    graph = graph or capture_request(block)
    eng.mirror.resync()
    out: List[int] = []
    budget = eng._kv_budget() - 2 * M8
    rounds = accepted = 0
    pending = [_launch(eng, graph)]
    while pending:
        if len(pending) < 2 and len(out) + len(pending) < max_new:
            pending.append(_launch(eng, graph))
        words = eng.mirror.wait(pending.pop(0))
        if words[Ctl.STATUS] != 0 or words[Ctl.COMMIT_COUNT] <= 0:
            for gen in pending:
                eng.mirror.wait(gen)
            raise RuntimeError(f"DFlash round failed: status {words[Ctl.STATUS]}")
        n = words[Ctl.COMMIT_COUNT]
        toks = words[Ctl.EMITTED : Ctl.EMITTED + n]
        rounds += 1
        accepted += n
        stop = False
        for t in toks:
            out.append(t)
            if (eos is not None and t == eos) or len(out) >= max_new:
                stop = True
                break
        if on_tokens:
            on_tokens(toks)
        if stop or words[Ctl.COMMITTED_LEN] >= budget:
            for gen in pending:
                eng.mirror.wait(gen)
            break
    if stats is not None:
        stats.update(rounds=rounds, accept_mean=accepted / max(rounds, 1))
    return out[:max_new]


def _launch(eng, graph) -> int:
    graph.replay()
    return eng.mirror.next_gen()
