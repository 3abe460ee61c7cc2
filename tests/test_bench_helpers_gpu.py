"""``utils.bench.bench_graph`` and ``profile_pipeline`` on kernels whose duration is known: nodes that spin on
``%globaltimer`` for a given number of nanoseconds (``nexrt_null_node``).  The replay time must be the sum of the nodes
(within launch overheads), the L2-flushed form must agree with the back-to-back form, and the telescoping profile must
attribute each stage its own spin time and add up to the whole (reference bench.py:71-129,147-205)."""

import ctypes

import pytest
import torch

from nexrt_b200.ops import lib as L
from nexrt_b200.runtime.capture import graph_capture
from nexrt_b200.utils.bench import ClockSampler, bench_graph, profile_pipeline

pytestmark = pytest.mark.gpu


def _node(lib, ns, stream):
    L.check(lib.nexrt_null_node(4, 64, 0, ns, 0, None, ctypes.c_void_p(stream.cuda_stream)), "null_node")


def test_bench_graph_times_known_nodes():
    lib = L.load()
    dev = torch.device("cuda", 0)
    side = torch.cuda.Stream(dev)
    spins = [20_000, 50_000, 30_000]                        # 100 us of work per replay
    with torch.cuda.stream(side):
        for ns in spins:
            _node(lib, ns, side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with graph_capture(g, side):
        for ns in spins:
            _node(lib, ns, side)
    plain = bench_graph(g, reps=20, warmup=3, device=dev, trials=3)
    assert len(plain["trials_ms"]) == 3 and plain["total_ms"] == pytest.approx(plain["ms_per_replay"] * 20)
    us = plain["ms_per_replay"] * 1e3
    assert 100.0 <= us < 160.0, us              # three kernel boundaries on top of the 100 us of spinning; slack for a busy host
    flushed = bench_graph(g, reps=10, warmup=2, device=dev, flush_l2=True)["ms_per_replay"] * 1e3
    assert 100.0 <= flushed < 220.0, flushed


def test_profile_pipeline_attributes_each_stage():
    lib = L.load()
    dev = torch.device("cuda", 0)
    spins = {"a": 40_000, "b": 10_000, "c": 25_000}
    made = []

    def stage(ns):
        def run():
            _node(lib, ns, torch.cuda.current_stream())
        return run

    for ns in spins.values():
        made.append(stage(ns))
    rows = profile_pipeline(made, list(spins), reps=20, warmup=3, device=dev)
    assert [r["stage"] for r in rows] == list(spins)
    for r, ns in zip(rows, spins.values()):
        assert abs(r["increment_us"] - ns / 1e3) < 15.0, (r, ns)
    assert rows[-1]["cumulative_us"] == pytest.approx(sum(r["increment_us"] for r in rows), rel=1e-6)


def test_clock_sampler_reports_a_summary():
    s = ClockSampler(0, period_ms=50).start()
    x = torch.randn(4096, 4096, device="cuda")
    for _ in range(20):
        x = x @ x * 1e-3
    torch.cuda.synchronize()
    out = s.stop()
    assert isinstance(out, dict)
    if out.get("samples"):
        assert out["sm_max_mhz"] >= out["sm_mhz"] > 0
