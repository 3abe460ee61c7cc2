"""Launch-environment checks and orderly termination for the serving workers.

The reference validates that the bridge runs as exactly eight single-node torchrun workers
(``sglang_prefill/process_supervisor.py:21-36``).  Here the tensor-parallel degree is a parameter
(1, 2, 4 or 8), a lone process without torchrun variables counts as TP=1, and the module also owns
the "terminate every rank" path used after a fatal invariant violation.
"""

from __future__ import annotations

import os
import signal
import sys
from typing import Mapping, Optional, Tuple

FATAL_EXIT_CODE = 2


def launch_geometry(tp_size: Optional[int] = None, env: Optional[Mapping[str, str]] = None) -> Tuple[int, int, int]:
    """Return ``(rank, world, local_rank)`` or raise ``ValueError`` if the launch is not one node of
    ``tp_size`` workers."""
    env = os.environ if env is None else env
    if "LOCAL_RANK" not in env:
        if tp_size not in (None, 1):
            raise ValueError(f"launch with torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node={tp_size}")
        return 0, 1, 0
    try:
        rank, world = int(env["RANK"]), int(env["WORLD_SIZE"])
        local, local_world = int(env["LOCAL_RANK"]), int(env.get("LOCAL_WORLD_SIZE", env["WORLD_SIZE"]))
    except (KeyError, ValueError) as error:
        raise ValueError(f"incomplete torchrun environment: {error}") from error
    if world not in (1, 2, 4, 8):
        raise ValueError(f"tensor-parallel degree must be 1, 2, 4 or 8, got {world}")
    if tp_size is not None and world != tp_size:
        raise ValueError(f"expected {tp_size} workers, torchrun started {world}")
    if local_world != world or rank != local or not 0 <= rank < world:
        raise ValueError(f"the server needs one node with {world} local workers (rank {rank}, local rank {local}, local world {local_world})")
    return rank, world, local


def terminate_group(reason: str, code: int = FATAL_EXIT_CODE, *, log=None, exit_fn=os._exit) -> None:
    """Fatal exit of this rank.  torchrun tears the other workers down when one exits non-zero, which
    is the collective stop the serving protocol relies on; stdio is flushed first because ``os._exit``
    skips interpreter shutdown."""
    (log or (lambda m: print(m, file=sys.stderr)))(f"@@ SERVE terminating all ranks: {reason}")
    for stream in (sys.stdout, sys.stderr):
        try:
            stream.flush()
        except (OSError, ValueError):
            pass
    exit_fn(code)


def install_signal_handlers(on_stop) -> None:
    """SIGTERM / SIGINT -> ``on_stop()`` once (lets the listen loop close its socket)."""
    fired = []

    def handler(signum, _frame):
        if not fired:
            fired.append(signum)
            on_stop()

    for sig in (signal.SIGTERM, signal.SIGINT):
        signal.signal(sig, handler)
