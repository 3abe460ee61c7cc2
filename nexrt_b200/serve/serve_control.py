"""Failure taxonomy and the collective success / reset / terminate policy of the server.

Policy of the reference (``nex_n2_5_pro/sglang_prefill/serve_control.py:31-251``): a request failure
may be *reset* (clear the cache session and every status latch, answer the client with an error,
keep serving) only if every rank reports a recoverable failure at the same lifecycle point;
anything that smells of a broken CUDA context or a broken process group, or any disagreement
between ranks, terminates all ranks.  There is no elastic recovery: a dead rank ends the group and
the launcher supervises lifetime.
"""

from __future__ import annotations

import enum
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


class LocalOutcome(enum.Enum):
    """What one rank saw when it ran the request, before the ranks compare notes."""

    DONE = "done"                  # returned a result
    RECOVERABLE = "recoverable"    # raised RecoverableRequestError
    FATAL_BACKEND = "fatal-backend"    # CUDA / NCCL / driver trouble: nothing can be agreed any more
    FATAL_UNKNOWN = "fatal-unknown"    # any other exception: state unknown, a reset could not be trusted


def _run_locally(request: Callable[[], object]):
    """Run ``request`` and classify how it ended: ``(outcome, result, error)``.  ``FatalTPInvariantError`` and
    ``FatalBackendError`` pass through untouched - they are verdicts already."""
    try:
        return LocalOutcome.DONE, request(), None
    except (FatalTPInvariantError, FatalBackendError):
        raise
    except RecoverableRequestError as error:
        return LocalOutcome.RECOVERABLE, None, error
    except Exception as error:  # noqa: BLE001 - classified below
        return (LocalOutcome.FATAL_BACKEND if is_fatal_backend_error(error) else LocalOutcome.FATAL_UNKNOWN), None, error


# what a fatal local outcome turns into (raised from the original error)
_FATAL_VERDICTS = {
    LocalOutcome.FATAL_BACKEND: (FatalBackendError, "fatal backend failure during request: {error!r}"),
    LocalOutcome.FATAL_UNKNOWN: (FatalTPInvariantError, "unexpected request failure cannot be reset safely: {error!r}"),
}


def execute_request_with_consensus(request: Callable[[], object], *, lifecycle_state: Callable[[], tuple],
                                   gather_outcome: Callable[[tuple], list], reset_request: Callable[[str], None]):
    """Run one request on this rank, then agree with the other ranks on what happened.

    Local verdicts that cannot be negotiated (backend failure, unknown exception) are raised at once.  Otherwise every
    rank contributes one compact record (failed or not, plus its cache lifecycle point); the group outcome is either
    "all fine" - the local result is returned, and a rank that failed alone is a broken invariant - or "reset", in which
    case ``reset_request(reason)`` runs on every rank and ``RequestResetError`` reports it to the caller."""
    outcome, result, error = _run_locally(request)
    if outcome in _FATAL_VERDICTS:
        verdict, template = _FATAL_VERDICTS[outcome]
        raise verdict(template.format(error=error)) from error
    failed_here = outcome is LocalOutcome.RECOVERABLE
    records = gather_outcome(failure_record(True if failed_here else None, *lifecycle_state()))
    group_outcome, _ = resolve_request_outcome(records)
    if group_outcome != "reset":
        if failed_here:
            raise FatalTPInvariantError(f"this rank failed but the group reports success: {records}")
        return result
    resolve_failure(records)       # raises when the ranks do not agree on where they failed
    reason = str(error) if failed_here else "collective request reset"
    reset_request(reason)
    raise RequestResetError(reason)


class _Reply:
    """Where rank 0 writes the answer of one socket request: the NDJSON event stream when the client asked for one,
    else a single JSON line on the connection.  Other ranks get a reply object that writes nothing."""

    def __init__(self, conn, event_stream, active: bool):
        self.conn, self.stream, self.active = conn, event_stream, active

    def _line(self, payload) -> None:
        self.conn.sendall((json.dumps(payload, ensure_ascii=False) + "\n").encode())

    def result(self, payload) -> None:
        if self.active:
            self.stream.finish(payload) if self.stream is not None else self._line(payload)

    def error(self, text: str) -> None:
        if self.active:
            self.stream.fail(text) if self.stream is not None else self._line({"error": text})

    def abandon(self) -> None:
        if self.active and self.stream is not None:
            self.stream.cancel()

    def release(self) -> None:
        if self.active and self.conn is not None:
            if self.stream is not None:
                self.stream.close()
            self.conn.close()


def dispatch_port_request(request: Callable[[], dict], *, tp_rank: int, conn, event_stream, report: list,
                          terminate_fatally: Callable, log_reset: Optional[Callable] = None):
    """Answer one socket request without ever leaving the ranks in different states: a result is sent and recorded, an
    agreed reset is answered with an error and serving goes on, anything else ends every rank through
    ``terminate_fatally`` (which must not return).  Only rank 0 touches the socket; it is always released."""
    reply = _Reply(conn, event_stream, active=tp_rank == 0)
    try:
        try:
            result = request()
        except RequestResetError as reset:
            if log_reset is not None:
                log_reset(reset)
            reply.error(repr(reset))
            return None
        except (KeyboardInterrupt, SystemExit):
            raise
        except BaseException as fatal:  # noqa: BLE001 - broken invariant, backend failure or a bug: all ranks must stop
            reply.abandon()
            terminate_fatally(fatal, None if event_stream is not None else conn)
            raise AssertionError("terminate_fatally returned")
        if reply.active:
            report.append(result)
        reply.result(result)
        return result
    finally:
        reply.release()
