"""Per-node cost of a captured graph of empty kernels: the floor under every step kernel.

    python -m nexrt_b200.utils.launch_floor [--nodes 64,128,256] [--grids 148,256] [--smem 0,40000] [--body-ns 0,2000]

Captures K empty nodes (``nexrt_null_node``: dependency wait, optional spin of ``body-ns`` on ``%globaltimer``, exit)
chained on one stream, launched exactly like the step kernels (programmatic dependent launch unless ``--no-pdl``), and
fits ``latency(K) = a + b K`` over the node counts: ``b`` is what one more kernel boundary costs in a replayed graph for
that grid / block / shared-memory footprint.  Same purpose as the reference's ``--scale`` mode
(``nex_n2_5_pro/decode_engine.py:549-630``).
"""

from __future__ import annotations

import argparse
import json

import torch


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--nodes", default="64,128,256")
    ap.add_argument("--grids", default="1,148,256")
    ap.add_argument("--block", type=int, default=256)
    ap.add_argument("--smem", default="0,40000")
    ap.add_argument("--body-ns", default="0,2000")
    ap.add_argument("--reps", type=int, default=50)
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--late-release", action="store_true", help="release dependents at the end of the node instead of at its start")
    a = ap.parse_args()
    from ..ops import lib as L
    from ..runtime.capture import graph_capture
    from .bench import bench_graph

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = L.load()
    if a.no_pdl:
        lib.nexrt_set_pdl(0)
    side = torch.cuda.Stream(device=dev)
    clk = torch.zeros(2, dtype=torch.int64, device=dev)     # SM cycles and nanoseconds of the last spinning node
    counts = [int(v) for v in a.nodes.split(",")]
    for grid in (int(v) for v in a.grids.split(",")):
        for smem in (int(v) for v in a.smem.split(",")):
            for body in (int(v) for v in a.body_ns.split(",")):
                times = []
                for k in counts:
                    def run():
                        for _ in range(k):
                            err = lib.nexrt_null_node(grid, a.block, smem, body, 0 if a.late_release else 1, clk.data_ptr() if body else None, side.cuda_stream)
                            if err:
                                raise RuntimeError(f"nexrt_null_node: cudaError {err}")
                    with torch.cuda.stream(side):
                        run()
                    torch.cuda.synchronize(dev)
                    g = torch.cuda.CUDAGraph()
                    with graph_capture(g, side):
                        run()
                    times.append(bench_graph(g, a.reps, warmup=5, device=dev)["ms_per_replay"] * 1e3)
                n = len(counts)
                mx, my = sum(counts) / n, sum(times) / n
                b = sum((x - mx) * (y - my) for x, y in zip(counts, times)) / sum((x - mx) ** 2 for x in counts)
                cyc, ns = clk.tolist()
                print(json.dumps({"grid": grid, "block": a.block, "smem": smem, "body_ns": body, "pdl": not a.no_pdl, "early_release": not a.late_release,
                                  "sm_mhz_in_graph": round(cyc / ns * 1e3, 1) if (body and ns) else None,
                                  "us_per_node": round(b, 3), "intercept_us": round(my - b * mx, 2), "us_total": [round(t, 1) for t in times]}), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
