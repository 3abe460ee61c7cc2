"""Prefill throughput of the engine's two prefill paths on one GPU: the 8-row steps and the wide chunks
(``prefill_wide.WidePrefill``), on a random-init model with the shard shapes of one rank of a ``--tp``-wide group
(no communication), ``--layers`` layers of the full geometry.

    python -m nexrt_b200.utils.bench_prefill --layers 8 --tp 8 --length 1024 --wide 64,128

Timing: CUDA events around a whole ``prefill`` call (host launches included: the 8-row path replays one captured
step per 8 tokens, the wide path one captured chunk), after one untimed call of the same kind; the prompt is
uniform-random ids.
"""

from __future__ import annotations

import argparse
import json

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--length", type=int, default=1024)
    ap.add_argument("--wide", default="64", help="comma list of wide chunk sizes to time (the 8-row path is always timed)")
    ap.add_argument("--shrunk", action="store_true")
    ap.add_argument("--no-rows", action="store_true", help="skip the 8-row path")
    a = ap.parse_args(argv)
    from ..config import full_config, shrunk_config
    from ..decode_engine import DecodeEngine
    from ..models.reference import synthetic_prompt
    from ..weights import random_rank_model

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = shrunk_config() if a.shrunk else full_config().truncated(a.layers)
    model = random_rank_model(cfg, a.tp, 0, dev)
    eng = DecodeEngine(0, 1, dev, ext=model, cfg=cfg, shape_tp=a.tp, max_rows=8, cache_len=a.length + 1024)
    prompt = synthetic_prompt(cfg.vocab, a.length, seed=1)
    eng.capture(8)

    def timed(wide: int) -> float:
        eng.prefill(prompt, chunk=8, wide=wide)      # warm-up: captures the chunk graph, fills caches
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.prefill(prompt, chunk=8, wide=wide)
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1)

    out = {"layers": cfg.n_layers, "tp_shapes": a.tp, "length": a.length, "paths": {}}
    cases = ([] if a.no_rows else [0]) + [int(w) for w in a.wide.split(",") if w]
    for wide in cases:
        ms = timed(wide)
        name = "rows8" if wide == 0 else f"wide{wide}"
        out["paths"][name] = {"ms": round(ms, 2), "tok_s": round(a.length / ms * 1e3, 1), "us_per_layer_per_token": round(ms * 1e3 / a.length / cfg.n_layers, 2)}
    out["status"] = eng.status_max()
    print(json.dumps(out), flush=True)
    return 0 if out["status"] == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
