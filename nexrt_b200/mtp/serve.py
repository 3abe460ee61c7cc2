"""Capture and serve loop of MTP speculative decoding.

Counterpart of ``nex_n2_5_pro/mtp/serve.py:39-138``: ``capture_round`` captures one whole round
(draft, 4-row verify, extend, control mirror) into a CUDA graph after warm-up; ``generate_mtp`` replays
it, queues round k+1 before reading round k from the host mirror, and emits the tokens each round
committed (``emitted[0 .. commit_count)``).
"""

from __future__ import annotations

from typing import Callable, List, Optional

import torch
from ..runtime.capture import graph_capture
import torch.distributed as dist

from ..runtime.rounds import Stops, consume_rounds
from .block import M_VERIFY, MtpDraft


def capture_round(mtp: MtpDraft, cp: bool = False, warmup: int = 3):
    eng = mtp.eng
    key = ("mtp", bool(cp))
    if key in eng.graphs:
        return eng.graphs[key]
    saved = eng._snapshot()
    y_saved = mtp.y_sel.clone()
    side = torch.cuda.Stream(device=eng.dev)
    side.wait_stream(torch.cuda.current_stream(eng.dev))
    with torch.cuda.stream(side):
        for _ in range(warmup):
            mtp.round(cp=cp)
    torch.cuda.current_stream(eng.dev).wait_stream(side)
    torch.cuda.synchronize(eng.dev)
    if eng.world > 1:
        dist.barrier(group=eng.group)
    g = torch.cuda.CUDAGraph()
    with graph_capture(g, side):
        mtp.round(cp=cp)
    eng._restore(saved)
    mtp.y_sel.copy_(y_saved)
    eng.graphs[key] = g
    if eng.world > 1:
        dist.barrier(group=eng.group)
    return g


def generate_mtp(mtp: MtpDraft, graph=None, max_new: int = 16, eos: Stops = None,
                 on_tokens: Optional[Callable[[List[int]], None]] = None, stats: Optional[dict] = None) -> List[int]:
    """Decode up to ``max_new`` tokens by replaying the round graph.  Returns the emitted tokens
    (the sequence is exactly what plain greedy / sampled decode would emit: drafts only decide how
    many tokens a round commits).  ``eos``: a stop token id or several; ``stats`` receives ``rounds`` and ``accept_mean``."""
    return consume_rounds(mtp.eng, graph or capture_round(mtp), max_new, eos, on_tokens, stats, reserve=2 * M_VERIFY, what="MTP round")
