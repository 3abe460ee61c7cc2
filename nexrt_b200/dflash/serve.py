"""Capture and serve loop of DFlash speculative decoding (reference ``nex_n2_5_pro/dflash/serve.py``:
``capture_request`` ``:29-45``, ``generate_dflash`` ``:48-121``)."""

from __future__ import annotations

from typing import Callable, List, Optional

import torch
from ..runtime.capture import graph_capture
import torch.distributed as dist

from ..runtime.rounds import Stops, consume_rounds
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


def generate_dflash(block: DFlashBlock, graph=None, max_new: int = 16, eos: Stops = None,
                    on_tokens: Optional[Callable[[List[int]], None]] = None, stats: Optional[dict] = None) -> List[int]:
    """Decode up to ``max_new`` tokens by replaying the request's round graph (``eos``: a stop token id or several)."""
    return consume_rounds(block.eng, graph or capture_request(block), max_new, eos, on_tokens, stats, reserve=2 * M8, what="DFlash round")
