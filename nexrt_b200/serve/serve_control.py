"""Failure taxonomy and the collective success / reset / terminate policy of the server.

Policy of the reference (``nex_n2_5_pro/sglang_prefill/serve_control.py:31-251``): a request failure
may be *reset* (clear the cache session and every status latch, answer the client with an error,
keep serving) only if every rank reports a recoverable failure at the same lifecycle point;
anything that smells of a broken CUDA context or a broken process group, or any disagreement
between ranks, terminates all ranks.  There is no elastic recovery: a dead rank ends the group and
the launcher supervises lifetime.
"""

from __future__ import annotations

import json
from typing import Callable, Optional

from .cache_consensus import (FatalTPInvariantError, RecoverableRequestError, failure_record, resolve_failure,
                              resolve_request_outcome)


class FatalBackendError(RuntimeError):
    """CUDA / NCCL / driver level failure: the process group cannot be trusted any more."""


class RequestResetError(RuntimeError):
    """The request failed, every rank agreed, state was reset; the server keeps running."""


class CacheReusePolicyError(ValueError):
    """A request asked for prompt-cache reuse where it is not offered."""


_FATAL_TYPE_MARKERS = ("cuda", "nccl", "c10d", "distbackenderror", "distnetworkerror")
_FATAL_TEXT_MARKERS = (
    "cudaerror=", "cuda error:", "cuda runtime error", "cuda driver error", "cuda initialization error", "cuda context",
    "context is destroyed", "context has been destroyed", "device-side assert", "illegal memory access",
    "unspecified launch failure", "processgroupnccl", "nccl error", "nccl communicator", "ncclunhandled", "c10d error",
)


def cache_key_for_request(cache_key, *, speculative: bool):
    """Prompt-cache reuse is offered on the plain decode path only."""
    if speculative and cache_key is not None:
        raise CacheReusePolicyError("cache reuse is not offered with MTP / DFlash decode; omit cache_key")
    return None if speculative else cache_key


def is_fatal_backend_error(error: BaseException) -> bool:
    """Typed fatal errors, exception types from the CUDA / c10d stack, or their well-known messages.
    The bare word "collective" is deliberately not a marker."""
    if isinstance(error, FatalBackendError):
        return True
    name = f"{type(error).__module__}.{type(error).__qualname__}".lower()
    if any(m in name for m in _FATAL_TYPE_MARKERS):
        return True
    text = str(error).lower()
    return any(m in text for m in _FATAL_TEXT_MARKERS)


def clear_request_statuses(engine, *speculative_blocks) -> None:
    """Zero every request-scoped failure latch: control-block status, LL channel state."""
    from ..runtime.control import Ctl

    engine.ctx.ctl[Ctl.STATUS] = 0
    for blk in speculative_blocks:
        for name in ("dctl", "cctl"):
            t = getattr(blk, name, None)
            if t is not None:
                t[Ctl.STATUS] = 0


def reset_failed_request(reason: str, *, cache, runtime_state: dict, engine, speculative_blocks=(), synchronize: Callable[[], None]) -> None:
    """Reset after a failure that all ranks have agreed is recoverable."""
    try:
        synchronize()
        cache.invalidate(reason, force=True)
        runtime_state["active_lease"] = None
        runtime_state["runtime_session"] = None
        clear_request_statuses(engine, *speculative_blocks)
        synchronize()
    except Exception as error:  # noqa: BLE001 - any failure while resetting is fatal
        raise FatalBackendError(f"failed to reset request state after {reason}: {error!r}") from error


def execute_request_with_consensus(request: Callable[[], object], *, lifecycle_state: Callable[[], tuple],
                                   gather_outcome: Callable[[tuple], list], reset_request: Callable[[str], None]):
    """Run one request on this rank, then agree with the other ranks on what happened."""
    local_error: Optional[BaseException] = None
    result = None
    try:
        result = request()
    except FatalTPInvariantError:
        raise
    except RecoverableRequestError as error:
        local_error = error
    except Exception as error:  # noqa: BLE001
        if isinstance(error, FatalBackendError):
            raise
        if is_fatal_backend_error(error):
            raise FatalBackendError(f"fatal backend failure during request: {error!r}") from error
        raise FatalTPInvariantError(f"unexpected request failure cannot be reset safely: {error!r}") from error
    generation, phase, active_generation, kind = lifecycle_state()
    rows = gather_outcome(failure_record(True if local_error is not None else None, generation, phase, active_generation, kind))
    outcome, _ = resolve_request_outcome(rows)
    if outcome == "reset":
        resolve_failure(rows)
        reason = str(local_error or "collective request reset")
        reset_request(reason)
        raise RequestResetError(reason)
    if local_error is not None:
        raise FatalTPInvariantError(f"this rank failed but the group reports success: {rows}")
    return result


def dispatch_port_request(request: Callable[[], dict], *, tp_rank: int, conn, event_stream, report: list,
                          terminate_fatally: Callable, log_reset: Optional[Callable] = None):
    """Answer one socket request without ever leaving the ranks in different states."""

    def send_line(payload) -> None:
        conn.sendall((json.dumps(payload, ensure_ascii=False) + "\n").encode())

    try:
        result = request()
        if tp_rank == 0:
            report.append(result)
            if event_stream is not None:
                event_stream.finish(result)
            else:
                send_line(result)
        return result
    except RequestResetError as error:
        if log_reset is not None:
            log_reset(error)
        if tp_rank == 0:
            if event_stream is not None:
                event_stream.fail(repr(error))
            else:
                send_line({"error": repr(error)})
        return None
    except BaseException as error:  # noqa: BLE001 - fatal invariant, backend failure or anything unexpected
        if isinstance(error, (KeyboardInterrupt, SystemExit)):
            raise
        if tp_rank == 0 and event_stream is not None:
            event_stream.cancel()
        terminate_fatally(error, None if event_stream is not None else conn)
        raise AssertionError("terminate_fatally returned")
    finally:
        if tp_rank == 0 and conn is not None:
            if event_stream is not None:
                event_stream.close()
            conn.close()
