"""Prefill throughput of the engine's two prefill paths on one GPU: the 8-row steps and the wide chunks
(``prefill_wide.WidePrefill``), on a random-init model with the shard shapes of one rank of a ``--tp``-wide group
(no communication), ``--layers`` layers of the full geometry; under ``torchrun`` the ranks form a real tensor-parallel
group instead and the in-kernel all-reduces run.

    python -m nexrt_b200.utils.bench_prefill --layers 8 --tp 8 --length 1024 --wide 64,128

Timing: CUDA events around a whole ``prefill`` call (host launches included: the 8-row path replays one captured
step per 8 tokens, the wide path one captured chunk), after one untimed call of the same kind; the prompt is
uniform-random ids.  ``--stages T`` instead replays the captured wide chunk of ``T`` rows with one stage stubbed out at a
time and prints what each stage adds to the chunk (timing attribution only: a chunk without a stage is not a prefill; without
the norm or the router every row routes to expert 0, the skip list then empties the expert products, and the figure printed
for those three stages is the experts' cost, not theirs).
"""

from __future__ import annotations

import argparse
import json

import torch


class _Skip:
    """The kernel library with the launches that ``pred(name, args)`` selects replaced by no-ops."""

    def __init__(self, lib, pred):
        self._lib, self._pred = lib, pred

    def __getattr__(self, name):
        f = getattr(self._lib, name)
        if not name.startswith("nexrt_"):
            return f
        pred = self._pred
        return lambda *args: 0 if pred(name, args) else f(*args)


def stage_costs(eng, T: int, replays: int = 10) -> dict:
    """Time of one captured chunk, and the time each stage adds to it (chunk time minus the time without the stage)."""
    from .. import prefill_wide
    from ..models.reference import synthetic_prompt
    from ..ops import tc_gemm

    cfg, spec, dev = eng.cfg, eng.spec, eng.dev
    real = eng.ctx.lib
    fronts = {spec.gdn_front_rows, spec.attn_front_rows}
    stages = {
        "all": lambda n, a: False,
        "norm_rows": lambda n, a: n == "nexrt_norm_rows",
        "front_gemms": lambda n, a: (n == "nexrt_tc_gemm_fp8" and a[7] in fronts and a[7] != cfg.hidden) or (n == "nexrt_tc_gemm_fp8_ex" and a[12] == 0 and a[13] is None),
        "gdn_chunk": lambda n, a: n == "nexrt_gdn_chunk",
        "kv_publish": lambda n, a: n == "nexrt_kv_publish",
        "attn_front_tail": lambda n, a: n == "nexrt_attn_front_tail",
        "attn_decode": lambda n, a: n == "nexrt_attn_decode",
        "gate_quant": lambda n, a: n in ("nexrt_gdn_gate_quant", "nexrt_act_quant"),
        "out_gemms": lambda n, a: n == "nexrt_tc_gemm_fp8" and a[7] == cfg.hidden,
        "residual": lambda n, a: n == "nexrt_planes_residual",
        "router_gemms": lambda n, a: n == "nexrt_tc_gemm_bf16_ex",
        "router_topk": lambda n, a: n == "nexrt_moe_router_topk",
        "expert_up_gemm": lambda n, a: n == "nexrt_tc_gemm_fp8_ex" and a[12] == 0 and a[13] is not None,
        "dense_act": lambda n, a: n == "nexrt_moe_dense_act",
        "expert_down_gemm": lambda n, a: n == "nexrt_tc_gemm_fp8_ex" and a[12] != 0,
    }
    prompt = synthetic_prompt(cfg.vocab, 2 * T, seed=1)
    out = {}
    for name, pred in stages.items():
        proxy = _Skip(real, pred)
        eng.ctx.lib = proxy
        tc_gemm.lib = lambda proxy=proxy: proxy
        eng.reset(first_token=prompt[0])
        wp = prefill_wide.WidePrefill(eng, T)
        wp.run(prompt)                      # eager pass, capture, two replays
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            wp.graph.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        out[name] = e0.elapsed_time(e1) * 1e3 / replays
        del wp
    eng.ctx.lib = real
    from ..ops.lib import load

    tc_gemm.lib = load
    full = out.pop("all")
    return {"chunk_us": round(full, 1), "adds_us": {k: round(full - v, 1) for k, v in out.items()}}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--length", type=int, default=1024)
    ap.add_argument("--wide", default="64", help="comma list of wide chunk sizes to time (the 8-row path is always timed)")
    ap.add_argument("--terms", default="1", help="comma list of activation term counts of the wide path (1 = one e4m3 plane, 3 = the exact split)")
    ap.add_argument("--shrunk", action="store_true")
    ap.add_argument("--no-rows", action="store_true", help="skip the 8-row path")
    ap.add_argument("--stages", type=int, default=0, help="chunk size whose stages are timed by leaving one out at a time")
    a = ap.parse_args(argv)
    from ..config import full_config, shrunk_config
    from ..decode_engine import DecodeEngine
    from ..models.reference import synthetic_prompt
    from ..weights import random_rank_model

    # under torchrun (WORLD_SIZE > 1) the ranks form a real tensor-parallel group of that size: the all-reduces of both
    # paths run (in-kernel LL packets), times are the maximum over the ranks
    import os

    import torch.distributed as dist

    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    cfg = shrunk_config() if a.shrunk else full_config().truncated(a.layers)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        a.tp = world
        model = random_rank_model(cfg, world, rank, dev)
        eng = DecodeEngine(rank, world, dev, ext=model, cfg=cfg, max_rows=8, cache_len=max(a.length + 1024, 16 * a.stages))
    else:
        model = random_rank_model(cfg, a.tp, 0, dev)
        eng = DecodeEngine(0, 1, dev, ext=model, cfg=cfg, shape_tp=a.tp, max_rows=8, cache_len=max(a.length + 1024, 16 * a.stages))
    if a.stages:
        res = stage_costs(eng, a.stages)
        res.update({"layers": cfg.n_layers, "tp_shapes": a.tp, "rows": a.stages, "status": eng.status_max()})
        print(json.dumps(res), flush=True)
        return 0
    prompt = synthetic_prompt(cfg.vocab, a.length, seed=1)
    if not a.no_rows:
        eng.capture(8)      # the 8-row path replays a captured step; without it the prompt's tail runs eagerly

    def timed(wide: int) -> float:
        eng.prefill(prompt, chunk=8, wide=wide)      # warm-up: captures the chunk graph, fills caches
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.prefill(prompt, chunk=8, wide=wide)
        e1.record()
        torch.cuda.synchronize(dev)
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    out = {"layers": cfg.n_layers, "tp_shapes": a.tp, "ranks": world, "length": a.length, "paths": {}}
    cases = ([] if a.no_rows else [(0, 1)]) + [(int(w), int(t)) for t in a.terms.split(",") if t for w in a.wide.split(",") if w]
    for wide, terms in cases:
        eng.wide_terms = terms
        ms = timed(wide)
        name = "rows8" if wide == 0 else (f"wide{wide}" if terms == 1 else f"wide{wide}x{terms}")
        out["paths"][name] = {"ms": round(ms, 2), "tok_s": round(a.length / ms * 1e3, 1), "us_per_layer_per_token": round(ms * 1e3 / a.length / cfg.n_layers, 2)}
    out["status"] = eng.status_max()
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if out["status"] == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
