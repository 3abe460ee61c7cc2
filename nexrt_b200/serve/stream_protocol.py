"""Token streaming: incremental detokenisation and a bounded, non-blocking NDJSON writer.

Behaviour of the reference (``nex_n2_5_pro/sglang_prefill/stream_protocol.py:51-292``): text is
emitted only when it can no longer change (a byte-fallback sequence is never split), stop tokens end
the visible stream, and the writer thread owns the socket so the decode callback never blocks on a
slow client - when the backlog is full the client is dropped, not the decode loop.

Wire format, one JSON object per line: ``{"type":"delta","text":…}`` ..., then exactly one of
``{"type":"done", …result}`` or ``{"type":"error","error":…}``.
"""

from __future__ import annotations

import json
import queue
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

    def _compact(self) -> None:
        if len(self.window) <= self.max_tail_tokens:
            return
        full = _decode(self.tokenizer, self.window)
        for keep in range(min(self.max_tail_tokens, len(self.window) - 1), 0, -1):
            cut = len(self.window) - keep
            head, tail = _decode(self.tokenizer, self.window[:cut]), _decode(self.tokenizer, self.window[cut:])
            if head + tail == full and not head.endswith(REPLACEMENT) and len(head) <= self.sent:
                del self.window[:cut]
                self.sent -= len(head)
                return
        raise RuntimeError(f"tokenizer has no exact incremental split within {self.max_tail_tokens} retained tokens")

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
            self._compact()
        return "".join(parts)

    def finish(self) -> str:
        text = _decode(self.tokenizer, self.window) if self.window else ""
        out = text[self.sent :]
        self.window.clear()
        self.sent = 0
        return out


_END = object()


class BridgeStreamWriter:
    """Owns the client socket; drains a bounded queue of events on its own thread."""

    DEFAULT_MAX_BACKLOG = 256
    DEFAULT_SHUTDOWN_TIMEOUT = 0.25
    DEFAULT_WRITE_TIMEOUT = 1.0

    def __init__(self, conn, tokenizer, stop_ids=(), *, max_backlog=None, shutdown_timeout=None, write_timeout=None, max_tail_tokens=None):
        self.conn = conn
        self.detok = IncrementalDetokenizer(tokenizer, stop_ids, max_tail_tokens=max_tail_tokens)
        backlog = self.DEFAULT_MAX_BACKLOG if max_backlog is None else int(max_backlog)
        if backlog < 2:
            raise ValueError("max_backlog must be >= 2")
        self.shutdown_timeout = self.DEFAULT_SHUTDOWN_TIMEOUT if shutdown_timeout is None else float(shutdown_timeout)
        wt = self.DEFAULT_WRITE_TIMEOUT if write_timeout is None else float(write_timeout)
        if self.shutdown_timeout <= 0 or wt <= 0:
            raise ValueError("writer timeouts must be > 0")
        self.q: "queue.Queue" = queue.Queue(maxsize=backlog)
        self.lock = threading.Lock()
        self.disconnected = threading.Event()
        self.stopped = threading.Event()
        self.finished = False
        self.error: Optional[BaseException] = None
        try:
            conn.settimeout(wt)
        except (AttributeError, OSError):
            pass
        self.thread = threading.Thread(target=self._drain, name="bridge-stream-writer", daemon=True)
        self.thread.start()

    # ---- producer side (decode callback; never blocks) ---------------------------------------------
    def _put(self, item, final: bool = False) -> bool:
        with self.lock:
            if self.finished or self.disconnected.is_set():
                return False
            try:
                self.q.put_nowait(item)
            except queue.Full:
                self.disconnected.set()
                if final:
                    self.finished = True
                return False
            if final:
                self.finished = True
            return True

    def event(self, payload: dict) -> bool:
        return self._put(("event", dict(payload)))

    def tokens(self, token_ids: Iterable[int]) -> bool:
        return self._put(("tokens", tuple(int(t) for t in token_ids)))

    def finish(self, result: dict) -> bool:
        return self._put(("finish", dict(result)), final=True)

    def fail(self, error) -> bool:
        return self._put(("error", str(error)), final=True)

    def cancel(self) -> None:
        """Drop queued output and free a writer stuck in a send."""
        with self.lock:
            self.finished = True
            self.disconnected.set()
            try:
                self.q.put_nowait(_END)
            except queue.Full:
                pass
        self._shutdown()

    def close(self) -> bool:
        """Stop the writer within a fixed deadline; returns False if it had to be abandoned."""
        with self.lock:
            if not self.finished:
                self.finished = True
                try:
                    self.q.put_nowait(_END)
                except queue.Full:
                    self.disconnected.set()
        self.thread.join(self.shutdown_timeout)
        if self.thread.is_alive():
            self.disconnected.set()
            self._shutdown()
            self.thread.join(self.shutdown_timeout)
        return not self.thread.is_alive()

    # ---- consumer side -----------------------------------------------------------------------------
    def _shutdown(self) -> None:
        try:
            self.conn.shutdown(socket.SHUT_RDWR)
        except (AttributeError, OSError):
            pass

    def _send(self, payload: dict) -> None:
        self.conn.sendall((json.dumps(payload, ensure_ascii=False) + "\n").encode())

    def _drain(self) -> None:
        try:
            while not self.disconnected.is_set():
                try:
                    item = self.q.get(timeout=self.shutdown_timeout)
                except queue.Empty:
                    if self.finished:
                        break
                    continue
                if item is _END:
                    break
                kind, payload = item
                if kind == "tokens":
                    text = self.detok.push(payload)
                    if text:
                        self._send({"type": "delta", "text": text})
                elif kind == "finish":
                    text = self.detok.finish()
                    if text:
                        self._send({"type": "delta", "text": text})
                    payload.pop("generated_text", None)
                    payload["type"] = "done"
                    self._send(payload)
                    break
                elif kind == "error":
                    self._send({"type": "error", "error": payload})
                    break
                else:
                    self._send(payload)
        except Exception as error:  # noqa: BLE001 - a broken client only ends this stream
            self.error = error
            self.disconnected.set()
        finally:
            self.stopped.set()
