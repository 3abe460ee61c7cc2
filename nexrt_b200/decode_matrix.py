"""Whole-step decode benchmark over a sweep of context lengths.

The weights are loaded and the step graph captured once; per length the engine either installs a
saved prefill state (``prefill_state_<layers>_<L>/`` written by :mod:`nexrt_b200.extract_state`) or
prefills a deterministic prompt itself, compares a teacher-forced greedy stream with ``golden.pt``
when there is one (a mismatch is tolerated only as a near tie of the engine's own logits), and times
free-running graph replay: median of ``--trials`` device-timed runs of ``--reps`` replays, MAX over
the ranks.  Same procedure as the reference's ``decode_matrix.py:44-243``.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 -m nexrt_b200.decode_matrix \
        --lengths 512,1024,2048,4096,8192 --steps 32
"""

from __future__ import annotations

import argparse
import json
import os
from pathlib import Path
from typing import Dict, List, Optional

import torch

NEAR_TIE_LOGIT_GAP = 0.30


def compare_with_golden(engine, golden: List[int], steps: int, graph) -> Dict:
    """Teacher-forced comparison: feed the golden token at every step, compare the engine's argmax."""
    from .runtime.control import Ctl

    mismatches, near = [], 0
    n = min(steps, len(golden) - 1)
    for i in range(n):
        engine.ctx.ctl[Ctl.PENDING] = int(golden[i])
        engine.mirror.resync()
        graph.replay()
        torch.cuda.synchronize(engine.dev)
        got = int(engine.ctx.ctl[Ctl.PENDING].item())
        if got != int(golden[i + 1]):
            gap = engine.logit_gap(got, int(golden[i + 1]))
            if gap is not None and gap <= NEAR_TIE_LOGIT_GAP:
                near += 1
            else:
                mismatches.append((i, got, int(golden[i + 1]), gap))
    return {"compared": n, "near_ties": near, "mismatches": mismatches}


def run_length(engine, graph, length: int, state_root: Optional[Path], steps: int, reps: int, trials: int, warmup: int) -> Dict:
    from .extract_state import load_state, make_prompt, state_dir
    from .utils.bench import bench_graph

    row: Dict = {"L": length}
    sdir = state_dir(state_root, engine.cfg.n_layers, length) if state_root else None
    if sdir is not None and (sdir / f"prefill_state_rank{engine.rank}.pt").is_file():
        load_state(engine, sdir)
        row["source"] = "state"
        gpath = sdir / "golden.pt"
        if gpath.is_file():
            snap = engine._snapshot()
            row["golden"] = compare_with_golden(engine, torch.load(gpath, weights_only=False)["tokens"], steps, graph)
            engine._restore(snap)
    else:
        engine.prefill(make_prompt(length, engine.cfg.vocab))
        row["source"] = "prefill"
    snap = engine._snapshot()
    t = bench_graph(graph, reps, warmup=warmup, device=engine.dev, group=engine.group, trials=trials)
    row["us_per_tok"] = round(1e3 * t["ms_per_replay"], 2)
    row["tok_s"] = round(1e3 / t["ms_per_replay"], 2)
    row["status"] = engine.status_max()
    engine._restore(snap)
    return row


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--lengths", default="512,1024,2048,4096,8192")
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=15)
    ap.add_argument("--reps", type=int, default=300)
    ap.add_argument("--trials", type=int, default=3)
    ap.add_argument("--state-root", type=Path, default=None)
    ap.add_argument("--layers", type=int, default=int(os.environ.get("NEXRT_NLAYERS", "60")))
    ap.add_argument("--layers-dir", default=None)
    ap.add_argument("--cp", action="store_true")
    ap.add_argument("--json", default=None, help="write the table here as JSON lines")
    a = ap.parse_args(argv)
    import torch.distributed as dist

    from .config import full_config
    from .decode_engine import DecodeEngine
    from .sampling import GREEDY
    from .serve.process_supervisor import launch_geometry
    from .weights import load_rank_model, random_rank_model

    rank, world, local = launch_geometry()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lengths = [int(x) for x in a.lengths.split(",") if x]
    cfg = full_config().truncated(a.layers)
    model = (load_rank_model(cfg, a.layers_dir, world, rank, dev, cp=a.cp) if a.layers_dir
             else random_rank_model(cfg, world, rank, dev))
    eng = DecodeEngine(rank, world, dev, cp=a.cp, ext=model, cfg=cfg, max_rows=8, cache_len=max(lengths) + a.reps * (a.trials + 1) + a.warmup + 1024)
    eng.head.set_sampling_config(0, *GREEDY)
    if a.state_root is not None:
        eng.head.enable_logits()      # before capture: the graph bakes the logits pointer
    eng.prefill([1, 2, 3, 4])
    graph = eng.capture(1, cp=False, warmup=a.warmup)
    rows = []
    for L in lengths:
        g = graph
        if a.cp and L >= eng.cp_threshold:
            g = eng.capture(1, cp=True, warmup=a.warmup)
        row = run_length(eng, g, L, a.state_root, a.steps, a.reps, a.trials, a.warmup)
        rows.append(row)
        if rank == 0:
            print("@@ MATRIX " + json.dumps(row), flush=True)
    if rank == 0 and a.json:
        with open(a.json, "w") as f:
            for row in rows:
                f.write(json.dumps(row) + "\n")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
