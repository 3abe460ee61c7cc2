"""Kernel timeline of one replayed decode step, from timestamps the kernels take themselves.

    NEXRT_TRACE_BUILD=1 python -m nexrt_b200.utils.trace_step --layers 8 --tp 8 --ctx 1024
    NEXRT_TRACE_BUILD=1 torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 -m nexrt_b200.utils.trace_step --layers 8

Needs the timeline variant of the library (``NEXRT_TRACE_BUILD=1``: the same sources compiled with
``-DNEXRT_TRACE``).  In it thread 0 of every CTA of every step kernel stores ``%globaltimer`` at its entry, after
its programmatic-dependency wait, at a kernel-specific midpoint (own product done, before the ticket or the
all-reduce) and at its exit.  This tool replays the captured whole-step graph with the trace buffer installed,
groups the records into launches and prints, per launch in execution order:

    entry  first CTA entered            (how early programmatic launch put the kernel on the machine)
    wait   first / last CTA past its dependency wait
    mid    last CTA at its midpoint
    exit   last CTA gone
    cost   exit minus the previous kernel's exit   (the kernel's share of the serial step)
    hand   first CTA past its wait minus the previous kernel's exit   (the hand-off latency)

and a per-kind average.  The counterpart in the reference is the cumulative-prefix profiler
(``nex_n2_5_pro/bench.py:147-205``); that one attributes time to stages, this one shows where inside a stage it goes.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
from collections import defaultdict

import torch
import torch.distributed as dist

KIND_NAMES = ["embed", "gdn_front", "gdn_core", "oproj_ar", "router", "moe_l1", "moe_l2_ar", "attn_front", "attn_decode", "head", "step_end",
              "tc_moe_l1", "tc_moe_l2", "tc_rows", "tc_router", "helper"]


def collect(buf: torch.Tensor, kinds: int, slots: int, words: int):
    """Launch records from the raw buffer: list of dicts sorted by exit time."""
    host = buf.cpu()
    cursors = host[:kinds].tolist()
    recs = host[kinds:].view(kinds, slots, words)
    launches = []
    for k in range(kinds):
        n = min(int(cursors[k]), slots)
        if n == 0:
            continue
        r = recs[k, :n]
        order = torch.argsort(r[:, 1])
        r = r[order]
        # a kind may hold launches of different grids (the helper kernels): records are grouped, in entry order, with the
        # others of their own grid size until a launch is complete
        grids = (r[:, 0] >> 32).tolist()
        open_groups, groups = {}, []
        for i, gsz in enumerate(grids):
            open_groups.setdefault(gsz, []).append(i)
            if len(open_groups[gsz]) == gsz:
                groups.append(open_groups.pop(gsz))
        for idxs in groups:
            g = r[torch.tensor(idxs)]
            grid = g.shape[0]
            t0, t1, t2, t3 = g[:, 1], g[:, 2], g[:, 3], g[:, 4]
            extras = [int(g[:, j][g[:, j] > 0].max()) if (g[:, j] > 0).any() else 0 for j in range(5, words)]
            t2v = t2[t2 > 0]
            launches.append({
                "raw": g.clone(),
                "kind": k, "grid": grid, "entry": int(t0.min()), "entry_last": int(t0.max()),
                "wait_first": int(t1[t1 > 0].min()) if (t1 > 0).any() else int(t0.min()), "wait_last": int(t1.max()),
                "mid_last": int(t2v.max()) if t2v.numel() else 0, "exit_first": int(t3[t3 > 0].min()) if (t3 > 0).any() else 0, "exit": int(t3.max()), "extras": extras,
            })
    launches.sort(key=lambda d: d["exit"])
    return launches


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--tp", type=int, default=8, help="shard shapes when run on one GPU")
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--cp", action="store_true", help="context-parallel attention arm (needs a world whose ranks share kv heads)")
    ap.add_argument("--show-layers", type=int, default=4, help="print the launches of the first N layers in full")
    ap.add_argument("--json", default="")
    ap.add_argument("--phases", default="", help="kernel name: print per-CTA durations between its stamps (mean / max over CTAs and launches)")
    a = ap.parse_args()
    if os.environ.get("NEXRT_TRACE_BUILD", "0") != "1":
        raise SystemExit("set NEXRT_TRACE_BUILD=1: the timeline lives in the trace variant of the library")
    from ..config import full_config
    from ..decode_engine import DecodeEngine
    from ..ops import lib as L
    from ..serve.process_supervisor import launch_geometry
    from ..weights import random_rank_model

    rank, world, local = launch_geometry()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = L.load()
    kinds, slots, words = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib.nexrt_trace_layout(ctypes.byref(kinds), ctypes.byref(slots), ctypes.byref(words))
    kinds, slots, words = kinds.value, slots.value, words.value
    cfg = full_config().truncated(a.layers)
    tp = world if world > 1 else a.tp
    model = random_rank_model(cfg, tp, rank if world > 1 else 0, dev, cp=a.cp)
    eng = DecodeEngine(rank, world, dev, cp=a.cp, ext=model, cfg=cfg, shape_tp=None if world > 1 else a.tp, max_rows=max(a.rows, 1), cache_len=a.ctx + 4096)
    if a.cp and not eng.cp:
        raise SystemExit("--cp: this world has no context-parallel group (every rank owns whole kv heads)")
    eng.reset(first_token=1, committed_len=a.ctx)
    eng.set_rows(list(range(1, a.rows + 1)))
    eng.set_forced_commit(a.rows)
    buf = torch.zeros(kinds + kinds * slots * words, dtype=torch.int64, device=dev)
    if lib.nexrt_set_trace(buf.data_ptr()) != 0:
        raise SystemExit("the loaded library is not the trace variant")
    graph = eng.capture(a.rows, cp=a.cp)   # its eager warm-up steps install the buffer address in every translation unit
    for _ in range(10):
        graph.replay()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    buf.zero_()
    torch.cuda.synchronize(dev)
    graph.replay()
    graph.replay()                         # the second replay is the one in steady state (its first kernels overlap the first's tail)
    torch.cuda.synchronize(dev)
    launches = collect(buf, kinds, slots, words)
    lib.nexrt_set_trace(None)
    status = eng.status_max()
    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0
    # keep the second replay: everything after the first step_end
    ends = [i for i, l in enumerate(launches) if l["kind"] == KIND_NAMES.index("step_end")]
    if len(ends) >= 2:
        launches = launches[ends[0] + 1 : ends[1] + 1]
    t_base = launches[0]["wait_first"]
    per_kind = defaultdict(lambda: defaultdict(list))
    prev_exit = launches[0]["wait_first"]
    n_per_layer = 6
    print(f"timeline of one step: rows={a.rows} ctx={a.ctx} layers={cfg.n_layers} world={world} tp-shapes={tp} status={status}")
    print(f"{'#':>4} {'kernel':12} {'grid':>5} {'entry':>8} {'entryN':>8} {'wait0':>8} {'wait1':>8} {'mid':>8} {'exit0':>8} {'exit':>8} | {'cost':>6} {'hand':>6} {'body':>6} {'tail':>6} | extras (last CTA at marks 4..7)")
    out_rows = []
    for i, l in enumerate(launches):
        rel = lambda t: (t - t_base) / 1e3 if t else float("nan")
        cost = (l["exit"] - prev_exit) / 1e3
        hand = (l["wait_first"] - prev_exit) / 1e3
        body = ((l["mid_last"] or l["exit"]) - l["wait_first"]) / 1e3
        tail = (l["exit"] - (l["mid_last"] or l["exit"])) / 1e3
        name = KIND_NAMES[l["kind"]]
        for key, v in (("cost", cost), ("hand", hand), ("body", body), ("tail", tail), ("lead", (prev_exit - l["entry"]) / 1e3)):
            per_kind[name][key].append(v)
        row = {"i": i, "kernel": name, "grid": l["grid"], "entry": rel(l["entry"]), "wait_first": rel(l["wait_first"]), "wait_last": rel(l["wait_last"]),
               "mid_last": rel(l["mid_last"]), "exit_first": rel(l["exit_first"]), "exit": rel(l["exit"]), "cost": cost, "hand": hand, "body": body, "tail": tail}
        out_rows.append(row)
        if i < 1 + n_per_layer * a.show_layers or i >= len(launches) - 2:
            ex = " ".join(f"{rel(t):8.2f}" for t in l["extras"] if t)
            print(f"{i:4d} {name:12} {l['grid']:5d} {row['entry']:8.2f} {rel(l['entry_last']):8.2f} {row['wait_first']:8.2f} {row['wait_last']:8.2f} {row['mid_last']:8.2f} "
                  f"{row['exit_first']:8.2f} {row['exit']:8.2f} | {cost:6.2f} {hand:6.2f} {body:6.2f} {tail:6.2f} | {ex}")
        prev_exit = l["exit"]
    total = (launches[-1]["exit"] - t_base) / 1e3
    print(f"step: {total:.1f} us from the first kernel's wait to the last exit, {len(launches)} launches")
    print(f"{'kernel':12} {'n':>4} {'cost':>7} {'hand':>7} {'body':>7} {'tail':>7} {'lead':>7}   (mean us; lead = how long before the previous exit the first CTA was resident)")
    for name, d in per_kind.items():
        n = len(d["cost"])
        mean = lambda k: sum(d[k]) / n
        print(f"{name:12} {n:4d} {mean('cost'):7.2f} {mean('hand'):7.2f} {mean('body'):7.2f} {mean('tail'):7.2f} {mean('lead'):7.2f}")
    if a.phases:
        # per-CTA time between consecutive stamps of one kernel kind: the launch table above shows the LAST CTA at each mark,
        # which mixes different CTAs; this is what one CTA spends in each phase
        k = KIND_NAMES.index(a.phases)
        order = {"gdn_front": [1, 2, 5, 7, 3, 6, 4], "moe_l1": [1, 5, 2, 6, 7, 8, 4], "moe_l2_ar": [1, 2, 5, 6, 7, 3, 4],
                 "attn_decode": [1, 2, 5, 6, 3, 7, 8, 4], "head": [1, 2, 3, 5, 6, 7, 4]}.get(a.phases, [1, 2, 3, 4])
        names = {1: "entry", 2: "wait", 3: "mid", 4: "exit", 5: "m4", 6: "m5", 7: "m6", 8: "m7"}
        rows = torch.cat([l["raw"] for l in launches[1 + n_per_layer :] if l["kind"] == k])      # skip the first layer (cold)
        print(f"per-CTA phase durations of {a.phases} ({rows.shape[0]} CTA records), us: mean / p50 / max")
        prev = None
        for col in order:
            t = rows[:, col].double()
            if prev is not None:
                ok = (t > 0) & (rows[:, prev] > 0)
                d = (t[ok] - rows[:, prev].double()[ok]) / 1e3
                if d.numel():
                    print(f"  {names[prev]:>6} -> {names[col]:<6} {d.mean():7.2f} {d.median():7.2f} {d.max():7.2f}")
            if (t > 0).any():
                prev = col
    for l in launches:
        l.pop("raw", None)
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"rows": out_rows, "total_us": total, "world": world, "layers": cfg.n_layers, "ctx": a.ctx}, f)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
