"""The in-kernel all-reduce alone: against the link's one-hop latency floor and against NCCL.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29511 -m nexrt_b200.utils.bench_allreduce

Per row count M (1, 4, 8 by default; ``4096 * M`` fp32 values, the payload of every reduce site of a step) it times

    ll-mc     the production epilogue (``csrc/epilogue.cuh``) publishing through the NVSwitch multicast alias
    ll-peer   the same epilogue with one store per peer instead
    nccl      ``ncclAllReduce`` of the same fp32 buffer

each as ``--calls`` back-to-back launches inside one captured graph (time per call = graph time / calls, CUDA events,
max over ranks), plus, for the two packet forms, the time one CTA spends between its first store and its last peer
value (``%globaltimer`` inside the kernel, median over CTAs and calls): the first figure contains the kernel boundary,
the second is the exchange itself.  Two ranks that run such calls back to back keep whatever skew they start with (up
to one hop): the rank that is ahead waits skew + hop, the other hop - skew, so the exchange is quoted as the slowest
rank's median and as the mean of the ranks' medians.  The yardstick is a two-rank ping-pong of one tagged packet (``hop``: half the
measured round trip, unicast and multicast): an all-reduce is one hop when every rank publishes at the same moment, so
``floor / exchange`` is the fraction of the latency floor the protocol reaches.

The reference times its fused reduce kernels against NCCL only (``nex_n2_5_pro/decode_engine.py:259-276``).
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading

import torch
import torch.distributed as dist


def _max_over_ranks(value: float, dev, world: int) -> float:
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _mean_over_ranks(value: float, dev, world: int) -> float:
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t)
    return float(t.item()) / world


def _time_graph(graph, reps: int, dev, world: int) -> float:
    """Mean milliseconds of one replay, max over ranks."""
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize(dev)
    return _max_over_ranks(a.elapsed_time(b) / reps, dev, world)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", default="1,4,8")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--calls", type=int, default=64, help="all-reduces per captured graph")
    ap.add_argument("--reps", type=int, default=50)
    ap.add_argument("--pingpong", type=int, default=2000, help="round trips of the latency-floor kernel")
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    from ..ops import lib as L
    from ..ops.lib import check, ptr
    from ..parallel.channel import LLChannel
    from ..serve.process_supervisor import launch_geometry

    rank, world, local = launch_geometry()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = L.load()
    H = a.hidden
    ch = LLChannel(dev, world, rank, 8 * H, group=None)
    peer_struct = ch.variant(multicast=False)          # same inbox, one store per peer
    forms = [("ll-mc", ch.struct)] if ch.multicast else []
    forms.append(("ll-peer", peer_struct))
    stream = torch.cuda.Stream(dev)
    out = {"world": world, "hidden": H, "calls": a.calls, "multicast": ch.multicast, "backend": ch.buf.backend, "rows": {}}

    def sp():
        return ctypes.c_void_p(stream.cuda_stream)

    # ---- the latency floor: one packet there and back between ranks 0 and 1 -------------------------------------
    if world > 1:
        pp = torch.zeros(2, dtype=torch.int64, device=dev)
        tag0 = 0x40000000
        for name, use_mc in (("unicast", 0), ("multicast", 1)):
            if use_mc and not ch.multicast:
                continue
            best = None
            for _ in range(3):
                dist.barrier()
                with torch.cuda.stream(stream):
                    check(lib.nexrt_ll_pingpong(ctypes.byref(ch.struct), 0, 1, tag0, a.pingpong, use_mc, ptr(pp), sp()), "pingpong")
                stream.synchronize()
                tag0 += a.pingpong
                ns, done = (int(v) for v in pp.tolist())
                hop = ns / max(done, 1) / 2 / 1e3 if rank in (0, 1) else 0.0
                hop = _max_over_ranks(hop, dev, world)
                best = hop if best is None else min(best, hop)
            out[f"hop_us_{name}"] = best
        ch.reset()
        torch.cuda.synchronize(dev)
        dist.barrier()

    # ---- the all-reduce forms -------------------------------------------------------------------------------------
    for M in [int(v) for v in a.rows.split(",")]:
        partial = torch.randn(M, H, dtype=torch.float32, device=dev)
        x = torch.zeros(M, H, dtype=torch.bfloat16, device=dev)
        stamps = torch.zeros(a.calls, H // 16, dtype=torch.int64, device=dev)
        row = {}
        for name, st in forms if world > 1 else []:
            def body(with_stamps: bool):
                for i in range(a.calls):
                    check(lib.nexrt_ll_allreduce_bench(ptr(partial), ptr(x), M, H, ctypes.byref(st), i, ptr(stamps[i]) if with_stamps else None, sp()),
                          "ll_allreduce_bench")
                check(lib.nexrt_ll_seq_advance(ptr(ch.seq), a.calls, sp()), "seq_advance")
            graphs = {}
            for with_stamps in (False, True):
                with torch.cuda.stream(stream):
                    body(with_stamps)                      # eager once (loads the kernels before capture)
                    stream.synchronize()
                    dist.barrier()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        body(with_stamps)
                graphs[with_stamps] = g
            ms = _time_graph(graphs[False], a.reps, dev, world)
            _time_graph(graphs[True], 5, dev, world)
            inner = stamps.double().flatten() / 1e3
            row[name] = {"us_per_call": ms * 1e3 / a.calls, "exchange_us_p50": _max_over_ranks(float(inner.median()), dev, world),
                         "exchange_us_p50_mean": _mean_over_ranks(float(inner.median()), dev, world),
                         "exchange_us_max": _max_over_ranks(float(inner.max()), dev, world)}
            # the sum is the sum: every rank holds the same bits
            want = partial.clone()
            dist.all_reduce(want)
            row[name]["max_abs_err"] = float((x.float() - want).abs().max())
            row[name]["status"] = int(ch.status.item())
        if world > 1:
            buf = partial.clone()
            with torch.cuda.stream(stream):
                dist.all_reduce(buf)
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    for _ in range(a.calls):
                        dist.all_reduce(buf)
            row["nccl"] = {"us_per_call": _time_graph(g, a.reps, dev, world) * 1e3 / a.calls}
        out["rows"][str(M)] = row
    if rank == 0:
        floor = min(v for k, v in out.items() if k.startswith("hop_us_")) if world > 1 else None
        print(f"world {world}  multicast {out['multicast']}  symmetric memory: {out['backend']}")
        if floor is not None:
            print("one-hop latency floor (ping-pong round trip / 2): " + ", ".join(f"{k[7:]} {v:.2f} us" for k, v in out.items() if k.startswith("hop_us_")))
            print(f"{'rows':>4} {'form':8} {'us/call':>8} {'p50 max/mean':>13} {'max':>7} {'floor/exchange':>15} {'vs nccl':>8} {'err':>9} status")
            for M, row in out["rows"].items():
                nccl = row["nccl"]["us_per_call"]
                for name, r in row.items():
                    if name == "nccl":
                        print(f"{M:>4} {name:8} {nccl:8.2f}")
                        continue
                    r["floor_fraction"] = floor / r["exchange_us_p50_mean"] if r["exchange_us_p50_mean"] > 0 else None
                    print(f"{M:>4} {name:8} {r['us_per_call']:8.2f} {r['exchange_us_p50']:6.2f}/{r['exchange_us_p50_mean']:6.2f} {r['exchange_us_max']:7.2f} {r['floor_fraction']:15.2f} "
                          f"{nccl / r['us_per_call']:7.1f}x {r['max_abs_err']:9.2e} {r['status']}")
        print(json.dumps(out))
        if a.json:
            with open(a.json, "w") as f:
                json.dump(out, f)
    if world > 1:
        # the captured NCCL graphs go first: tearing the communicator down under a live graph that holds its kernels can
        # block for good, and a benchmark that printed its result must not hold the GPUs
        g = graphs = None
        torch.cuda.synchronize(dev)
        dist.barrier()
        sys.stdout.flush()
        threading.Timer(20.0, os._exit, (0,)).start()
        dist.destroy_process_group()
        os._exit(0)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
