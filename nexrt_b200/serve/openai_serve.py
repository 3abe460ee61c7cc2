"""OpenAI-compatible HTTP facade in front of the bridge socket.

Endpoints (same surface as the reference's ``sglang_prefill/openai_serve.py:408-710``):
``GET /health``, ``GET /v1/models``, ``GET /v1/models/<id>``, ``POST /v1/completions`` and
``POST /v1/chat/completions`` (JSON reply or Server-Sent Events when ``stream`` is true, with an
optional usage chunk under ``stream_options.include_usage``).  The engine serves one request at a
time, so the facade holds a single slot: a second request waits for ``--queue-timeout`` seconds and
is then refused with 429.  Controls the engine cannot honour (``n > 1``, custom ``stop`` strings,
penalties, logprobs, tools) are refused with 400 rather than ignored; per-request sampling is
forwarded only when the facade was started with ``--forward-sampling``.

The translation is a pair of pure functions (:func:`to_bridge_request`, :func:`to_openai_reply`) so it
can be tested without sockets; the HTTP part is a thin ``http.server`` handler.
"""

from __future__ import annotations

import argparse
import json
import threading
import time
import uuid
from dataclasses import dataclass, field
from http import HTTPStatus
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Callable, Dict, Iterator, Optional
from urllib.parse import unquote, urlsplit

from . import bridge_client

# a control is accepted only when absent or set to a value that means "off"
_OFF_VALUES = {
    "frequency_penalty": (0, 0.0, None), "presence_penalty": (0, 0.0, None), "repetition_penalty": (1, 1.0, None),
    "logprobs": (False, None, 0), "top_logprobs": (None, 0), "logit_bias": (None, {}), "tools": (None, []), "tool_choice": (None, "none"),
    "functions": (None, []), "response_format": (None, {"type": "text"}), "best_of": (None, 1), "echo": (None, False), "suffix": (None, ""),
    "min_p": (None, 0, 0.0),
}
_METRIC_KEYS = ("ttft_s", "prefill_s", "decode_us_per_tok", "accept_mean", "rounds", "cache", "forced_prefill", "mode", "consensus_ms")


class ApiError(Exception):
    def __init__(self, message: str, *, param: Optional[str] = None, status: HTTPStatus = HTTPStatus.BAD_REQUEST, kind: str = "invalid_request_error"):
        super().__init__(message)
        self.message, self.param, self.status, self.kind = message, param, status, kind

    def body(self) -> Dict:
        return {"error": {"message": self.message, "type": self.kind, "param": self.param, "code": None}}


def _int(value, name: str, minimum: Optional[int] = None) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise ApiError(f"{name} must be an integer", param=name)
    if minimum is not None and value < minimum:
        raise ApiError(f"{name} must be >= {minimum}", param=name)
    return value


def wants_usage_chunk(body: Dict) -> bool:
    opts = body.get("stream_options")
    if opts is None:
        return False
    if not body.get("stream", False):
        raise ApiError("stream_options requires stream=true", param="stream_options")
    if not isinstance(opts, dict):
        raise ApiError("stream_options must be an object", param="stream_options")
    extra = sorted(set(opts) - {"include_usage"})
    if extra:
        raise ApiError(f"stream_options.{extra[0]} is not supported", param=f"stream_options.{extra[0]}")
    flag = opts.get("include_usage", False)
    if not isinstance(flag, bool):
        raise ApiError("stream_options.include_usage must be a boolean", param="stream_options.include_usage")
    return flag


def to_bridge_request(body, endpoint: str, *, forward_sampling: bool = False) -> Dict:
    """OpenAI request body -> bridge request (raises :class:`ApiError` with the offending ``param``)."""
    if not isinstance(body, dict):
        raise ApiError("request body must be a JSON object")
    for name, off in _OFF_VALUES.items():
        if name in body and (body[name] is True or not any(body[name] == v for v in off)):
            raise ApiError(f"{name} is not supported by this backend", param=name)
    if body.get("n", 1) != 1:
        raise ApiError("only n=1 is supported", param="n")
    if body.get("stop") is not None:
        raise ApiError("custom stop sequences are not supported; the model's stop tokens stay enabled", param="stop")
    if not isinstance(body.get("stream", False), bool):
        raise ApiError("stream must be a boolean", param="stream")
    wants_usage_chunk(body)
    out: Dict = {"max_new": _int(body.get("max_completion_tokens", body.get("max_tokens", 256)), "max_tokens", 1)}
    if body.get("stream", False):
        out["stream"] = True
    if endpoint == "chat":
        msgs = body.get("messages")
        if not isinstance(msgs, list) or not msgs or not all(isinstance(m, dict) and "role" in m and "content" in m for m in msgs):
            raise ApiError("messages must be a non-empty array of {role, content}", param="messages")
        out["messages"] = msgs
    else:
        prompt = body.get("prompt")
        if not isinstance(prompt, str) or not prompt:
            raise ApiError("prompt must be a non-empty string", param="prompt")
        out["text"] = prompt
    if body.get("seed") is not None:
        out["seed"] = _int(body["seed"], "seed", 0)
    if body.get("cache_key") is not None:
        if not isinstance(body["cache_key"], str) or not body["cache_key"]:
            raise ApiError("cache_key must be a non-empty string", param="cache_key")
        out["cache_key"] = body["cache_key"]
    for name in ("temperature", "top_p", "top_k"):
        if body.get(name) is not None:
            if not forward_sampling:
                raise ApiError("per-request sampling needs --forward-sampling", param=name)
            out[name] = body[name]
    return out


def finish_reason(result: Dict, requested: int) -> str:
    if result.get("stop_reason") == "eos":
        return "stop"
    return "length" if result.get("stop_reason") in ("length", "context") or len(result.get("tokens", ())) >= requested else "stop"


def usage(result: Dict) -> Dict:
    p, c = int(result.get("prompt_tokens", 0)), len(result.get("tokens", ()))
    return {"prompt_tokens": p, "completion_tokens": c, "total_tokens": p + c}


def check_bridge_result(result) -> Dict:
    if not isinstance(result, dict):
        raise ApiError("malformed backend reply", status=HTTPStatus.BAD_GATEWAY, kind="backend_error")
    if "error" in result:
        bad = str(result["error"]).startswith("bad request")
        raise ApiError(str(result["error"]), status=HTTPStatus.BAD_REQUEST if bad else HTTPStatus.BAD_GATEWAY,
                       kind="invalid_request_error" if bad else "backend_error")
    status = result.get("status", 0)
    if isinstance(status, bool) or not isinstance(status, int):
        raise ApiError("malformed backend reply: status is not an integer", status=HTTPStatus.BAD_GATEWAY, kind="backend_error")
    if status != 0:
        raise ApiError(f"backend reported device status {status}", status=HTTPStatus.BAD_GATEWAY, kind="backend_error")
    if not isinstance(result.get("tokens"), list):
        raise ApiError("backend reply has no tokens", status=HTTPStatus.BAD_GATEWAY, kind="backend_error")
    if not isinstance(result.get("generated_text", ""), str) or not isinstance(result.get("prompt_tokens", 0), int):
        raise ApiError("malformed backend reply: text / prompt_tokens", status=HTTPStatus.BAD_GATEWAY, kind="backend_error")
    return result


def to_openai_reply(endpoint: str, result: Dict, model: str, requested: int, request_id: Optional[str] = None) -> Dict:
    rid = request_id or uuid.uuid4().hex
    text, reason = result.get("generated_text", ""), finish_reason(result, requested)
    if endpoint == "chat":
        choice = {"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": reason}
        obj, rid = "chat.completion", f"chatcmpl-{rid}"
    else:
        choice = {"index": 0, "text": text, "finish_reason": reason, "logprobs": None}
        obj, rid = "text_completion", f"cmpl-{rid}"
    return {"id": rid, "object": obj, "created": int(time.time()), "model": model, "choices": [choice], "usage": usage(result),
            "nexrt_metrics": {k: result[k] for k in _METRIC_KEYS if k in result}}


def stream_chunk(endpoint: str, base: Dict, *, text: Optional[str] = None, role: bool = False, reason: Optional[str] = None) -> Dict:
    chunk = dict(base)
    if endpoint == "chat":
        delta: Dict = {}
        if role:
            delta["role"] = "assistant"
        if text is not None:
            delta["content"] = text
        chunk["choices"] = [{"index": 0, "delta": delta, "finish_reason": reason}]
    else:
        chunk["choices"] = [{"index": 0, "text": text or "", "finish_reason": reason, "logprobs": None}]
    return chunk


def primed(events: Iterator[Dict]) -> Iterator[Dict]:
    """Pull the first event now.  ``bridge_client.stream_request`` is a generator, so it connects only when first advanced:
    priming it before the status line goes out turns an unreachable backend into a 502 JSON reply instead of a broken
    200 stream."""
    return _Primed(events)


class _Primed:
    """An event stream whose first event has already been pulled; ``close()`` reaches the source (a generator that holds
    the backend socket), which ``itertools.chain`` would hide."""

    def __init__(self, events: Iterator[Dict]):
        self.source = iter(events)
        try:
            self.head = [next(self.source)]
        except StopIteration:
            self.head = []

    def __iter__(self):
        return self

    def __next__(self) -> Dict:
        if self.head:
            return self.head.pop()
        return next(self.source)

    def close(self) -> None:
        close = getattr(self.source, "close", None)
        if close:
            close()


def sse_events(endpoint: str, events: Iterator[Dict], model: str, requested: int, include_usage: bool, request_id: Optional[str] = None) -> Iterator[str]:
    """Bridge NDJSON events -> SSE ``data:`` lines (ending with ``[DONE]``)."""
    rid = request_id or uuid.uuid4().hex
    base = {"id": ("chatcmpl-" if endpoint == "chat" else "cmpl-") + rid, "object": "chat.completion.chunk" if endpoint == "chat" else "text_completion",
            "created": int(time.time()), "model": model}
    if include_usage:
        base["usage"] = None

    def line(obj) -> str:
        return "data: " + json.dumps(obj, ensure_ascii=False) + "\n\n"

    if endpoint == "chat":
        yield line(stream_chunk(endpoint, base, role=True))
    final = None
    source = iter(events)
    while True:
        try:
            ev = next(source)
        except StopIteration:
            break
        except (ConnectionError, OSError, TimeoutError, ValueError) as error:
            # the 200 header is out: a backend that dies in mid-stream is reported in-band, and the stream still ends with [DONE]
            yield line({"error": {"message": f"backend stream failed: {error}", "type": "backend_error", "param": None, "code": None}})
            yield "data: [DONE]\n\n"
            return
        kind = ev.get("type")
        if kind == "delta":
            yield line(stream_chunk(endpoint, base, text=ev.get("text", "")))
        elif kind == "done":
            try:
                device_status = int(ev.get("status", 0))
            except (TypeError, ValueError):
                device_status = -1
            if device_status != 0:     # a step latched a failure: what was streamed is not a completion, and it must not end like one
                yield line({"error": {"message": f"backend reported device status {ev.get('status')}", "type": "backend_error", "param": None, "code": None}})
                yield "data: [DONE]\n\n"
                return
            final = ev
            break
        elif kind == "error" or "error" in ev:
            yield line({"error": {"message": str(ev.get("error")), "type": "backend_error", "param": None, "code": None}})
            yield "data: [DONE]\n\n"
            return
    if final is None:
        yield line({"error": {"message": "backend stream ended early", "type": "backend_error", "param": None, "code": None}})
    else:
        yield line(stream_chunk(endpoint, base, reason=finish_reason(final, requested)))
        if include_usage:
            tail = dict(base, choices=[], usage=usage(final))
            yield line(tail)
    yield "data: [DONE]\n\n"


@dataclass
class FacadeState:
    model_name: str = "Nex-N2.5-Pro"
    backend_host: str = "127.0.0.1"
    backend_port: int = 9411
    backend_timeout: float = 1800.0
    queue_timeout: float = 30.0
    write_timeout: float = 30.0      # a streaming client that takes nothing for this long loses its stream (and frees the engine slot)
    forward_sampling: bool = False
    call: Callable = bridge_client.send_request
    stream: Callable = bridge_client.stream_request
    slot: threading.Semaphore = field(default_factory=lambda: threading.Semaphore(1))
    started: float = field(default_factory=time.time)


class Handler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"
    server_version = "nexrt-b200"

    @property
    def st(self) -> FacadeState:
        return self.server.state  # type: ignore[attr-defined]

    def log_message(self, fmt, *args):  # quiet by default
        pass

    def _json(self, status, body) -> None:
        data = json.dumps(body, ensure_ascii=False).encode()
        self.send_response(int(status))
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(data)))
        self.send_header("Access-Control-Allow-Origin", "*")
        self.end_headers()
        self.wfile.write(data)

    def do_OPTIONS(self):  # noqa: N802
        self.send_response(204)
        for k, v in (("Access-Control-Allow-Origin", "*"), ("Access-Control-Allow-Methods", "GET, POST, OPTIONS"),
                     ("Access-Control-Allow-Headers", "Content-Type, Authorization"), ("Content-Length", "0")):
            self.send_header(k, v)
        self.end_headers()

    def _model_card(self) -> Dict:
        return {"id": self.st.model_name, "object": "model", "created": int(self.st.started), "owned_by": "nexrt-b200"}

    def do_GET(self):  # noqa: N802
        path = urlsplit(self.path).path.rstrip("/") or "/"
        if path in ("/", "/health", "/healthz"):
            return self._json(200, {"status": "ok", "model": self.st.model_name})
        if path == "/v1/models":
            return self._json(200, {"object": "list", "data": [self._model_card()]})
        if path.startswith("/v1/models/"):
            if unquote(path[len("/v1/models/"):]) == self.st.model_name:
                return self._json(200, self._model_card())
            return self._json(404, ApiError("model not found", param="model", status=HTTPStatus.NOT_FOUND).body())
        self._json(404, ApiError("unknown path", status=HTTPStatus.NOT_FOUND).body())

    def do_POST(self):  # noqa: N802
        path = urlsplit(self.path).path.rstrip("/")
        endpoint = {"/v1/chat/completions": "chat", "/v1/completions": "text"}.get(path)
        try:
            if endpoint is None:
                raise ApiError("unknown path", status=HTTPStatus.NOT_FOUND)
            length = int(self.headers.get("Content-Length") or 0)
            if length <= 0 or length > (64 << 20):
                raise ApiError("a JSON body is required")
            try:
                body = json.loads(self.rfile.read(length).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as error:
                raise ApiError(f"invalid JSON: {error}") from error
            if isinstance(body, dict) and body.get("model") not in (None, self.st.model_name):
                raise ApiError(f"model {body.get('model')!r} is not served here", param="model", status=HTTPStatus.NOT_FOUND)
            req = to_bridge_request(body, endpoint, forward_sampling=self.st.forward_sampling)
            include_usage = wants_usage_chunk(body)
            if not self.st.slot.acquire(timeout=self.st.queue_timeout):
                raise ApiError("the engine is busy", status=HTTPStatus.TOO_MANY_REQUESTS, kind="rate_limit_error")
            try:
                if req.get("stream"):
                    return self._stream(endpoint, req, include_usage)
                result = check_bridge_result(self.st.call(req, self.st.backend_host, self.st.backend_port, self.st.backend_timeout))
                return self._json(200, to_openai_reply(endpoint, result, self.st.model_name, req["max_new"]))
            finally:
                self.st.slot.release()
        except ApiError as error:
            self._json(error.status, error.body())
        except (ConnectionError, OSError, TimeoutError) as error:
            self._json(502, ApiError(f"backend unreachable: {error}", status=HTTPStatus.BAD_GATEWAY, kind="backend_error").body())

    def _stream(self, endpoint: str, req: Dict, include_usage: bool) -> None:
        events = primed(self.st.stream(req, self.st.backend_host, self.st.backend_port, self.st.backend_timeout))   # may raise: do_POST answers 502
        self.send_response(200)
        self.send_header("Content-Type", "text/event-stream")
        self.send_header("Cache-Control", "no-cache")
        self.send_header("Connection", "close")
        self.send_header("Access-Control-Allow-Origin", "*")
        self.end_headers()
        self.close_connection = True
        # the engine slot is held while the stream runs: a reader that stalls must not hold it forever, so every write is
        # bounded, and whichever way the stream ends the backend connection is closed with it
        self.connection.settimeout(self.st.write_timeout)
        try:
            for chunk in sse_events(endpoint, events, self.st.model_name, req["max_new"], include_usage):
                self.wfile.write(chunk.encode())
                self.wfile.flush()
        except (BrokenPipeError, ConnectionResetError, TimeoutError, OSError):
            pass                      # the client went away or stopped reading: nothing more can be told to it
        finally:
            events.close()


class OpenAIServer(ThreadingHTTPServer):
    daemon_threads = True
    allow_reuse_address = True

    def __init__(self, address, state: FacadeState):
        super().__init__(address, Handler)
        self.state = state


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="OpenAI-compatible facade for the nexrt_b200 bridge")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--backend-host", default="127.0.0.1")
    p.add_argument("--backend-port", type=int, default=9411)
    p.add_argument("--backend-timeout", type=float, default=1800.0)
    p.add_argument("--queue-timeout", type=float, default=30.0)
    p.add_argument("--write-timeout", type=float, default=30.0, help="seconds a streaming client may stall before its stream is dropped")
    p.add_argument("--model-name", default="Nex-N2.5-Pro")
    p.add_argument("--forward-sampling", action="store_true")
    a = p.parse_args(argv)
    state = FacadeState(a.model_name, a.backend_host, a.backend_port, a.backend_timeout, a.queue_timeout, a.write_timeout, a.forward_sampling)
    with OpenAIServer((a.host, a.port), state) as srv:
        print(f"@@ OPENAI facade on http://{a.host}:{srv.server_address[1]} -> bridge {a.backend_host}:{a.backend_port}", flush=True)
        try:
            srv.serve_forever()
        except KeyboardInterrupt:
            pass
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
