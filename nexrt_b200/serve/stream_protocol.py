"""Token streaming: incremental detokenisation and a bounded, non-blocking NDJSON writer.

Behaviour of the reference (``nex_n2_5_pro/sglang_prefill/stream_protocol.py:51-292``): text is
emitted only when it can no longer change (a byte-fallback sequence is never split), stop tokens end
the visible stream, and the writer thread owns the socket so the decode callback never blocks on a
slow client - when the backlog is full the client is dropped, not the decode loop.

Wire format, one JSON object per line: ``{"type":"delta","text":…}`` ..., then exactly one of
``{"type":"done", …result}`` or ``{"type":"error","error":…}``.
"""

from __future__ import annotations

import collections
import contextlib
import enum
import json
import socket
import threading
from typing import Iterable, List, Optional, Sequence

REPLACEMENT = "�"


def visible_token_ids(token_ids: Iterable[int], stop_ids: Iterable[int] = ()) -> List[int]:
    stops = {int(s) for s in stop_ids}
    out: List[int] = []
    for t in token_ids:
        if int(t) in stops:
            break
        out.append(int(t))
    return out


def _decode(tokenizer, ids: Sequence[int]) -> str:
    return tokenizer.decode(list(ids), skip_special_tokens=False, clean_up_tokenization_spaces=False)


def decode_visible_text(tokenizer, token_ids, stop_ids=()) -> str:
    return _decode(tokenizer, visible_token_ids(token_ids, stop_ids))


class IncrementalDetokenizer:
    """Emits the longest prefix of the decoded text that later tokens cannot change.

    The retained token window is decoded as a whole; whatever precedes an incomplete byte sequence
    (a trailing U+FFFD) is final and is emitted.  The window is compacted at a token boundary where
    decoding prefix and suffix separately reproduces the joint decode exactly, so memory and work
    per token stay bounded (``max_tail_tokens``)."""

    DEFAULT_MAX_TAIL_TOKENS = 32

    def __init__(self, tokenizer, stop_ids=(), *, max_tail_tokens: Optional[int] = None):
        self.tokenizer = tokenizer
        self.stop_ids = {int(s) for s in stop_ids}
        self.max_tail_tokens = self.DEFAULT_MAX_TAIL_TOKENS if max_tail_tokens is None else int(max_tail_tokens)
        if self.max_tail_tokens < 1:
            raise ValueError("max_tail_tokens must be >= 1")
        self.window: List[int] = []
        self.sent = 0             # characters of decode(window) already emitted
        self.stop_seen = False

    @property
    def retained_tokens(self) -> int:
        return len(self.window)

    def _stable_text(self) -> str:
        text = _decode(self.tokenizer, self.window)
        end = len(text)
        while end > 0 and text[end - 1] == REPLACEMENT:
            end -= 1
        if end < self.sent:
            return ""
        out, self.sent = text[self.sent : end], end
        return out

    def _compact(self) -> str:
        """Bound the window.  A cut is exact when decoding the two parts separately gives the joint text: then the cut lies
        between two characters (or invalid sequences) and nothing that follows can change the head.  Preferred: an exact
        cut whose head is already out.  Otherwise an exact cut whose head still holds unsent characters - trailing
        replacement characters of bytes that turned out to be final - which are returned for emission.  A tokenizer with
        no exact cut inside the tail at all (one character spread over more tokens than the tail keeps) gets its window
        flushed as it decodes now: a stream never fails over its own bookkeeping."""
        if len(self.window) <= self.max_tail_tokens:
            return ""
        full = _decode(self.tokenizer, self.window)
        forced = None
        for keep in range(min(self.max_tail_tokens, len(self.window) - 1), 0, -1):
            cut = len(self.window) - keep
            head, tail = _decode(self.tokenizer, self.window[:cut]), _decode(self.tokenizer, self.window[cut:])
            if head + tail != full:
                continue
            if len(head) <= self.sent:
                del self.window[:cut]
                self.sent -= len(head)
                return ""
            if forced is None:
                forced = (cut, head)
        if forced is not None:
            cut, head = forced
            out = head[self.sent :]
            del self.window[:cut]
            self.sent = 0
            return out
        out = full[self.sent :]
        self.window.clear()
        self.sent = 0
        return out

    def push(self, token_ids: Iterable[int]) -> str:
        if self.stop_seen:
            return ""
        parts = []
        for t in token_ids:
            t = int(t)
            if t in self.stop_ids:
                self.stop_seen = True
                break
            self.window.append(t)
            piece = self._stable_text()
            if piece:
                parts.append(piece)
            piece = self._compact()
            if piece:
                parts.append(piece)
        return "".join(parts)

    def finish(self) -> str:
        text = _decode(self.tokenizer, self.window) if self.window else ""
        out = text[self.sent :]
        self.window.clear()
        self.sent = 0
        return out


class WriterState(enum.Enum):
    OPEN = "open"            # accepting output
    SEALED = "sealed"        # the terminal event (done / error) is queued, or close() was asked for: nothing more is accepted
    DROPPED = "dropped"      # the client is gone or too slow, or the request was cancelled: queued output is discarded


class BridgeStreamWriter:
    """Owns the client socket of a streaming request.

    Producers (the decode loop's token callback) append to a bounded deque under a condition variable and return at
    once; one writer thread pops, detokenises and sends.  Consecutive token events that wait behind a send are merged
    into one.  A backlog that still reaches its limit means the client cannot keep up: the stream is dropped, never the
    decode loop.  Exactly one terminal event (``done`` or ``error``) can be
    queued; ``close()`` waits a bounded time for the thread and shuts the socket down under it if it is stuck in a send.
    """

    DEFAULT_MAX_BACKLOG = 256
    DEFAULT_SHUTDOWN_TIMEOUT = 0.25
    DEFAULT_WRITE_TIMEOUT = 1.0

    def __init__(self, conn, tokenizer, stop_ids=(), *, max_backlog=None, shutdown_timeout=None, write_timeout=None, max_tail_tokens=None):
        self.conn = conn
        self.detok = IncrementalDetokenizer(tokenizer, stop_ids, max_tail_tokens=max_tail_tokens)
        self.max_backlog = int(self.DEFAULT_MAX_BACKLOG if max_backlog is None else max_backlog)
        self.shutdown_timeout = float(self.DEFAULT_SHUTDOWN_TIMEOUT if shutdown_timeout is None else shutdown_timeout)
        write_timeout = float(self.DEFAULT_WRITE_TIMEOUT if write_timeout is None else write_timeout)
        if self.max_backlog < 2:
            raise ValueError("the backlog needs room for at least one event and the terminal one")
        if min(self.shutdown_timeout, write_timeout) <= 0:
            raise ValueError("shutdown_timeout and write_timeout must be positive")
        self._pending: "collections.deque" = collections.deque()
        self._cv = threading.Condition()
        self._state = WriterState.OPEN
        self.stopped = threading.Event()          # set when the writer thread has left its loop
        self.error: Optional[BaseException] = None
        with contextlib.suppress(AttributeError, OSError):
            conn.settimeout(write_timeout)
        self.thread = threading.Thread(target=self._writer_loop, name="bridge-stream-writer", daemon=True)
        self.thread.start()

    @property
    def state(self) -> WriterState:
        return self._state

    @property
    def disconnected(self) -> bool:
        return self._state is WriterState.DROPPED

    # ---- producer side: never blocks -------------------------------------------------------------------
    def _offer(self, kind: str, payload, terminal: bool = False) -> bool:
        with self._cv:
            if self._state is not WriterState.OPEN:
                return False
            if kind == "tokens" and self._pending and self._pending[-1][0] == "tokens":
                # tokens that queue up behind a slow send travel as one longer delta: a client that is slow but alive
                # costs no backlog slots (a dead one is found by the write timeout), and the decode loop still never waits
                self._pending[-1] = ("tokens", self._pending[-1][1] + payload)
                return True
            if len(self._pending) >= self.max_backlog:
                self._state = WriterState.DROPPED
                self._pending.clear()
                self._cv.notify_all()
                return False
            self._pending.append((kind, payload))
            if terminal:
                self._state = WriterState.SEALED
            self._cv.notify_all()
            return True

    def event(self, payload: dict) -> bool:
        return self._offer("raw", dict(payload))

    def tokens(self, token_ids: Iterable[int]) -> bool:
        return self._offer("tokens", tuple(int(t) for t in token_ids))

    def finish(self, result: dict) -> bool:
        return self._offer("done", dict(result), terminal=True)

    def fail(self, error) -> bool:
        return self._offer("error", str(error), terminal=True)

    def cancel(self) -> None:
        """Discard queued output and free a writer thread that may be stuck in a send."""
        with self._cv:
            self._state = WriterState.DROPPED
            self._pending.clear()
            self._cv.notify_all()
        self._shutdown_socket()

    def close(self) -> bool:
        """Let the thread flush what is queued, within ``shutdown_timeout``; past that the socket is shut down under it.
        Returns False if the thread had to be abandoned."""
        with self._cv:
            if self._state is WriterState.OPEN:
                self._state = WriterState.SEALED
            self._cv.notify_all()
        self.thread.join(self.shutdown_timeout)
        if self.thread.is_alive():
            with self._cv:
                self._state = WriterState.DROPPED
                self._pending.clear()
                self._cv.notify_all()
            self._shutdown_socket()
            self.thread.join(self.shutdown_timeout)
        return not self.thread.is_alive()

    # ---- writer thread ---------------------------------------------------------------------------------------
    def _shutdown_socket(self) -> None:
        with contextlib.suppress(AttributeError, OSError):
            self.conn.shutdown(socket.SHUT_RDWR)

    def _write(self, payload: dict) -> None:
        self.conn.sendall((json.dumps(payload, ensure_ascii=False) + "\n").encode())

    def _next(self):
        """The next queued item, or None when there is nothing left to do."""
        with self._cv:
            while not self._pending:
                if self._state is not WriterState.OPEN:
                    return None
                self._cv.wait(self.shutdown_timeout)
            if self._state is WriterState.DROPPED:
                return None
            return self._pending.popleft()

    def _emit(self, kind: str, payload) -> bool:
        """Send one item; True when it was the terminal one."""
        if kind == "tokens":
            text = self.detok.push(payload)
            if text:
                self._write({"type": "delta", "text": text})
            return False
        if kind == "raw":
            self._write(payload)
            return False
        if kind == "done":
            tail = self.detok.finish()
            if tail:
                self._write({"type": "delta", "text": tail})
            body = {k: v for k, v in payload.items() if k != "generated_text"}   # the client has the text as deltas already
            body["type"] = "done"
            self._write(body)
        else:
            self._write({"type": "error", "error": payload})
        return True

    def _writer_loop(self) -> None:
        try:
            while True:
                item = self._next()
                if item is None or self._emit(*item):
                    break
        except Exception as error:  # noqa: BLE001 - a broken client only ends this stream
            self.error = error
            with self._cv:
                self._state = WriterState.DROPPED
                self._pending.clear()
        finally:
            self.stopped.set()
