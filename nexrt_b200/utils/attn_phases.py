"""Phase timestamps of the decode-attention kernel inside a replayed whole-step graph.

    python -m nexrt_b200.utils.attn_phases [--ctx 1024] [--tp 8] [--layers 4]

This tool times the TICKETED form of the kernel (a 148-CTA grid whose last CTA combines the split partials through a
workspace), which the step uses when thread-block clusters are switched off; it switches them off itself (bits 64 and
128 of the kernel-form mask).  The default cluster form is timed per CTA by ``utils/trace_step.py --phases``.

The kernel of kv head 0 writes ``%globaltimer`` at its phase boundaries into a 16-word ring
(``nexrt_set_attn_event_ring``): 0 start, 1 dependency wait over, 2 q/k normalised and rotated, 3 key
loop done, 4 warps merged and partial written, 5 ticket taken - and, in the CTA that took the last
ticket: 6 combine starts, 7 split scales ready, 9 partials summed, 10 output written, 8 end.  The
timestamps are printed relative to phase 0; they cost one store each and do not change the schedule.
"""

from __future__ import annotations

import argparse

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--layers", type=int, default=4)
    a = ap.parse_args()
    from ..config import full_config
    from ..decode_engine import DecodeEngine
    from ..ops import lib as L
    from ..weights import random_rank_model

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = full_config().truncated(a.layers)
    eng = DecodeEngine(0, 1, dev, ext=random_rank_model(cfg, a.tp, 0, dev), cfg=cfg, shape_tp=a.tp, max_rows=1, cache_len=a.ctx + 4096)
    eng.reset(first_token=1, committed_len=a.ctx)
    ring = torch.zeros(16, dtype=torch.int64, device=dev)
    lib = L.load()
    lib.nexrt_set_gemv_mode(255 & ~(64 | 128))
    lib.nexrt_set_attn_event_ring(ring.data_ptr())
    graph = eng.capture(1)
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    lib.nexrt_set_attn_event_ring(None)
    lib.nexrt_set_gemv_mode(255)
    r = ring.tolist()
    names = ["start", "wait_over", "qk_ready", "keys_done", "merged", "ticket", "combine_start", "scales_ready", "end", "summed", "stored"]
    order = [0, 1, 2, 3, 4, 5, 6, 7, 9, 10, 8]
    print(f"ctx={a.ctx} tp-shape={a.tp}: " + "  ".join(f"{names[i]}={(r[i] - r[0]) / 1e3:.2f}us" for i in order))


if __name__ == "__main__":
    main()
