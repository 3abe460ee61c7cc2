"""Stream capture with the Python garbage collector held still.

A CUDA stream capture in the default (global) error mode is invalidated by any call that frees device or pinned
memory while it runs.  The engine's buffers that come from the kernel library (symmetric inboxes, the host-mapped
control mirror) are freed with ``cudaFree`` / ``cudaFreeHost`` when their owner is collected, and the cyclic garbage
collector can decide to collect a dead engine in the middle of a capture that launches a few thousand kernels from
Python.  ``graph_capture`` therefore collects once before the capture starts and keeps the collector off until the
capture has ended.
"""

from __future__ import annotations

import contextlib
import gc

import torch


@contextlib.contextmanager
def graph_capture(graph: "torch.cuda.CUDAGraph", stream: "torch.cuda.Stream"):
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, stream=stream):
            yield
    finally:
        if was_enabled:
            gc.enable()
