"""Run a few eager decode steps of a random-init model at a chosen context length without a real
prefill (the committed length is simply set, the KV cache holds zeros): a timing fixture for
profilers, like the reference's ``slot[1]`` override (``nex_n2_5_pro/decode_engine.py:687-723``).

    python -m nexrt_b200.utils.profile_step --layers 4 --ctx 1024 --steps 3 --rows 1
"""

from __future__ import annotations

import argparse
import os

import torch


class _Without:
    """The kernel library with one entry point replaced by a no-op (timing attribution only)."""

    def __init__(self, lib, name: str):
        self._lib, self._name = lib, name

    def __getattr__(self, item):
        if item == self._name:
            return lambda *args: 0
        return getattr(self._lib, item)


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--layers", type=int, default=4)
    p.add_argument("--ctx", type=int, default=1024)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--rows", type=int, default=1)
    p.add_argument("--shrunk", action="store_true")
    p.add_argument("--tp", type=int, default=1, help="use the shard shapes of one rank of a tp-wide group (no communication)")
    p.add_argument("--graph", action="store_true", help="time captured-graph replays and print us/step")
    p.add_argument("--no-pdl", action="store_true")
    p.add_argument("--threads", type=int, default=0)
    p.add_argument("--leave-one-out", action="store_true", help="with --graph: re-capture with each kernel entry point stubbed out and print the time it adds to the step")
    a = p.parse_args()
    from ..config import full_config, shrunk_config
    from ..decode_engine import DecodeEngine
    from ..runtime.control import Ctl
    from ..weights import random_rank_model

    from ..ops import lib as L

    if a.no_pdl:
        L.load().nexrt_set_pdl(0)
    if a.threads:
        L.load().nexrt_set_gemv_threads(a.threads)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = shrunk_config() if a.shrunk else full_config().truncated(a.layers)
    model = random_rank_model(cfg, a.tp, 0, dev)
    eng = DecodeEngine(0, 1, dev, ext=model, cfg=cfg, shape_tp=a.tp, max_rows=max(a.rows, 1), cache_len=a.ctx + (a.steps + 16) * 12 * max(a.rows, 1) + 1024)   # room for every replay of every re-capture
    eng.reset(first_token=1, committed_len=a.ctx)
    eng.set_rows(list(range(1, a.rows + 1)))
    eng.set_forced_commit(a.rows)
    if a.graph:
        from .bench import bench_graph

        g = eng.capture(a.rows)
        r = bench_graph(g, a.steps, warmup=5, device=dev)
        full = r["ms_per_replay"] * 1e3
        print(f"rows={a.rows} ctx={a.ctx} layers={cfg.n_layers}: {full:.1f} us/step")
        if a.leave_one_out:
            real = eng.ctx.lib
            for name in ("nexrt_gdn_front", "nexrt_gdn_core", "nexrt_attn_front", "nexrt_attn_decode", "nexrt_oproj_allreduce", "nexrt_moe_router",
                         "nexrt_moe_l1", "nexrt_moe_l2_allreduce", "nexrt_lmhead_sample", "nexrt_rows_norm_split", "nexrt_tc_rows_gemm",
                         "nexrt_gdn_front_tail", "nexrt_tc_router_logits", "nexrt_moe_router_topk", "nexrt_tc_moe_l1", "nexrt_tc_moe_l2_allreduce",
                         "nexrt_lmhead_sample_from_logits"):
                eng.ctx.lib = _Without(real, name)
                eng.graphs.clear()
                t = bench_graph(eng.capture(a.rows), a.steps, warmup=5, device=dev)["ms_per_replay"] * 1e3
                print(f"  without {name:26s} {t:8.1f} us/step   (adds {full - t:6.1f} us)")
            eng.ctx.lib = real
    else:
        for _ in range(a.steps):
            eng.step(a.rows)
        torch.cuda.synchronize()
    print("status", int(eng.ctx.ctl[Ctl.STATUS]))


if __name__ == "__main__":
    main()
