"""Device-timed throughput of the tcgen05 GEMM on weight matrices larger than L2.

    python -m nexrt_b200.utils.bench_tc_gemm [--rows 65536] [--k 4096] [--tokens 16,64,128,256] [--small]

Prints one JSON line per case: time per call (CUDA events, after warm-up, inputs larger than L2 so every
call streams its weights from HBM), achieved weight bandwidth and FLOP rate, and the same product through
``torch.matmul`` on bf16 operands for scale.  ``--small`` runs one short case (for profiler captures).
"""

from __future__ import annotations

import argparse
import json

import torch

from ..ops.tc_gemm import act_quant, bf16_gemm, fp8_gemm
from ..quant import FP8


def timed(fn, reps: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--tokens", default="16,64,128,256")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--small", action="store_true")
    a = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    R, K = (40960, 4096) if a.small else (a.rows, a.k)
    tokens = [64] if a.small else [int(t) for t in a.tokens.split(",")]
    reps = 3 if a.small else a.reps
    g = torch.Generator(device=dev).manual_seed(0)
    wq = torch.randint(-60, 60, (R, K), device=dev, dtype=torch.int8, generator=g).view(FP8)       # small finite e4m3 codes
    sw = torch.rand(R // 128, K // 128, device=dev, generator=g) * 0.01 + 0.001
    wb = torch.randn(R, K, device=dev, generator=g).to(torch.bfloat16) * 0.02 if not a.small else None
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for T in tokens:
        x = torch.randn(T, K, device=dev, generator=g).to(torch.bfloat16)
        xq, sx = act_quant(x)
        out = torch.empty(T, R, dtype=torch.float32, device=dev)
        ms = timed(lambda: fp8_gemm(wq, sw, xq, sx, out=out, status=status), reps)
        row = {"case": "fp8_block_scaled", "T": T, "R": R, "K": K, "ms": round(ms, 4), "weight_GBs": round(R * K / ms / 1e6, 1),
               "TFLOPs": round(2 * T * R * K / ms / 1e9, 1)}
        if wb is not None:
            ms_b = timed(lambda: bf16_gemm(wb, x, out=out, status=status), reps)
            ms_t = timed(lambda: torch.matmul(x, wb.T), reps)
            row.update(bf16_ms=round(ms_b, 4), bf16_weight_GBs=round(2 * R * K / ms_b / 1e6, 1), bf16_TFLOPs=round(2 * T * R * K / ms_b / 1e9, 1),
                       torch_bf16_ms=round(ms_t, 4))
        row["status"] = int(status.item())
        print(json.dumps(row), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
