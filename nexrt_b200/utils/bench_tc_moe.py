"""Device-timed run of the tcgen05 expert kernels at the shard shapes of one rank of a TP=8 group.

    python -m nexrt_b200.utils.bench_tc_moe [--rows 8] [--reps 20] [--experts 512]

Every call streams its experts from HBM (the expert tables are far larger than L2 and each repetition uses a
different random routing).  Prints time, distinct experts, bytes streamed and the achieved bandwidth for the
gate/up kernel (one pass per distinct expert) and the down + all-reduce + residual kernel (single rank: the
packet exchange is skipped, the epilogue still does the residual update).  `--reps 2` keeps the run short for
profiler captures.
"""

from __future__ import annotations

import argparse
import json

import torch

from ..ops.lib import check, load, ptr
from ..parallel.channel import LLChannel
from ..quant import FP8


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--experts", type=int, default=512)
    ap.add_argument("--ksplit", type=int, default=2, help="CTAs per expert row tile along K in the gate/up product")
    a = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    H, I, E, S, M = 4096, 128, a.experts, 11, a.rows
    g = torch.Generator(device=dev).manual_seed(0)
    w13 = torch.randint(-60, 60, (E + 1, 2 * I, H), device=dev, dtype=torch.int8, generator=g).view(FP8)
    w13s = torch.rand(E + 1, 2 * I // 128, H // 128, device=dev, generator=g) * 0.01 + 0.001
    w2 = torch.randint(-60, 60, (E + 1, H, I), device=dev, dtype=torch.int8, generator=g).view(FP8)
    w2s = torch.rand(E + 1, H // 128, I // 128, device=dev, generator=g) * 0.01 + 0.001
    x = torch.randn(M, H, device=dev, generator=g).to(torch.bfloat16)
    gamma = torch.ones(H, device=dev)
    routings = [torch.stack([torch.cat([torch.randperm(E, device=dev, generator=g)[: S - 1], torch.tensor([E], device=dev)]) for _ in range(M)]).to(torch.int32)
                for _ in range(a.reps + 3)]
    wts = torch.rand(M, S, device=dev, generator=g) * 0.2
    gu = torch.zeros(a.ksplit, M, S, 2 * I, device=dev)
    p1 = torch.zeros(24, H, dtype=torch.uint8, device=dev)
    p2 = torch.zeros(24, S * I, dtype=torch.uint8, device=dev)
    ds = torch.zeros(8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ch = LLChannel(dev, 1, 0, 8 * H)
    lib, st = load(), torch.cuda.current_stream().cuda_stream

    def l1(ids):
        check(lib.nexrt_tc_moe_l1(ptr(x), ptr(gamma), ptr(w13), ptr(w13s), ptr(ids), ptr(gu), ptr(p1), H, I, S, M, E + 1, a.ksplit, 1e-6, 0, ptr(status), st), "l1")

    def l2(ids):
        check(lib.nexrt_tc_moe_l2_allreduce(ptr(gu), ptr(ids), ptr(wts), ptr(w2), ptr(w2s), ptr(x), ptr(p2), ptr(ds), H, I, S, M, E + 1, a.ksplit, ch.ref, 0,
                                            ptr(status), st), "l2")

    for ids in routings[:3]:
        l1(ids)
        l2(ids)
    torch.cuda.synchronize()
    out = {}
    for name, fn in (("gate_up", l1), ("down_allreduce", l2)):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for ids in routings[3:]:
            fn(ids)
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / a.reps * 1e3
    distinct = sum(len(torch.unique(r)) for r in routings[3:]) / a.reps
    b1, b2 = distinct * 2 * I * H, M * S * H * I
    print(json.dumps({"rows": M, "distinct_experts": round(distinct, 1),
                      "gate_up_us": round(out["gate_up"], 2), "gate_up_MB": round(b1 / 1e6, 1), "gate_up_GBs": round(b1 / out["gate_up"] / 1e3, 1),
                      "down_us": round(out["down_allreduce"], 2), "down_MB": round(b2 / 1e6, 1), "down_GBs": round(b2 / out["down_allreduce"] / 1e3, 1),
                      "note": "times include the activation split kernel launched with each GEMM", "status": int(status.item())}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
