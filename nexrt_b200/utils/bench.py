"""Timing helpers: captured-graph replay timing (max over ranks), telescoping per-stage profile,
clock sampling during a timed region.

Counterpart of the reference's ``bench_graph`` / ``profile_pipeline``
(``nex_n2_5_pro/bench.py:71-129,147-205``): replay timing is CUDA-event based on the launching
stream after warm-up, bracketed by a barrier and a device synchronise, and reduced with MAX over
the ranks; the pipeline profiler captures graphs of growing prefixes of the real step and
differences them so that the per-stage numbers add up to the whole step exactly.
"""

from __future__ import annotations

import statistics
import subprocess
import threading
from typing import Callable, Dict, List, Optional, Sequence

import torch
from ..runtime.capture import graph_capture
import torch.distributed as dist

L2_FLUSH_BYTES = 256 << 20


def _barrier(group=None) -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier(group=group)


def tp_max(value: float, device, group=None) -> float:
    """MAX of a host scalar over the ranks."""
    if not (dist.is_available() and dist.is_initialized()):
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def bench_graph(graph, reps: int, warmup: int = 10, device=None, group=None, flush_l2: bool = False, trials: int = 1) -> Dict:
    """Device time of ``reps`` back-to-back replays (or L2-flushed single replays)."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device) if flush_l2 else None
    for _ in range(warmup):
        graph.replay()
    results = []
    for _ in range(trials):
        torch.cuda.synchronize(device)
        _barrier(group)
        torch.cuda.synchronize(device)
        if flush is None:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(reps):
                graph.replay()
            stop.record()
            torch.cuda.synchronize(device)
            ms = start.elapsed_time(stop)
        else:
            ms = 0.0
            for _ in range(reps):
                flush.random_()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                graph.replay()
                stop.record()
                torch.cuda.synchronize(device)
                ms += start.elapsed_time(stop)
        _barrier(group)
        results.append(tp_max(ms, device, group))
    total = statistics.median(results)
    return {"total_ms": total, "ms_per_replay": total / reps, "trials_ms": results}


def profile_pipeline(stages: Sequence[Callable[[], None]], names: Sequence[str], reps: int = 50, warmup: int = 5, device=None,
                     group=None) -> List[Dict]:
    """Telescoping per-stage cost: graph k holds stages 0..k; stage k's cost is
    time(graph k) - time(graph k-1), so the column sums to the time of the whole step."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    prev, out = 0.0, []
    side = torch.cuda.Stream(device=device)
    for k in range(len(stages)):
        def run():
            for s in stages[: k + 1]:
                s()
        with torch.cuda.stream(side):
            for _ in range(2):
                run()
        torch.cuda.synchronize(device)
        g = torch.cuda.CUDAGraph()
        with graph_capture(g, side):
            run()
        t = bench_graph(g, reps, warmup, device, group)["ms_per_replay"]
        out.append({"stage": names[k], "cumulative_us": t * 1e3, "increment_us": (t - prev) * 1e3})
        prev = t
    return out


class ClockSampler:
    """Samples ``nvidia-smi`` SM clocks and throttle reasons while a timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.lines: List[str] = []
        self.proc: Optional[subprocess.Popen] = None
        self.thread: Optional[threading.Thread] = None

    def start(self) -> "ClockSampler":
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", f"-lms", str(self.period_ms),
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return self
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()
        return self

    def _pump(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> Dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return self.summary()

    def summary(self) -> Dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
