"""OpenAI facade: request translation, reply shaping, SSE stream, HTTP round trip against a fake bridge."""

import http.client
import json
import threading

import pytest

from nexrt_b200.serve.openai_serve import (ApiError, FacadeState, OpenAIServer, check_bridge_result, finish_reason, sse_events,
                                           to_bridge_request, to_openai_reply, wants_usage_chunk)

RESULT = {"tokens": [5, 6, 7], "generated_text": "abc", "status": 0, "stop_reason": "length", "prompt_tokens": 4, "cache": "hit",
          "ttft_s": 0.01, "decode_us_per_tok": 2500.0, "mode": "bs1"}


def test_translation_of_completions_and_chat():
    assert to_bridge_request({"prompt": "hi", "max_tokens": 3}, "text") == {"max_new": 3, "text": "hi"}
    r = to_bridge_request({"messages": [{"role": "user", "content": "hi"}], "max_completion_tokens": 9, "stream": True, "seed": 4, "cache_key": "k"}, "chat")
    assert r == {"max_new": 9, "stream": True, "messages": [{"role": "user", "content": "hi"}], "seed": 4, "cache_key": "k"}
    assert to_bridge_request({"prompt": "x"}, "text")["max_new"] == 256
    r = to_bridge_request({"prompt": "x", "temperature": 0.2, "top_p": 0.5, "top_k": 3}, "text", forward_sampling=True)
    assert (r["temperature"], r["top_p"], r["top_k"]) == (0.2, 0.5, 3)
    # values that mean "off" pass
    to_bridge_request({"prompt": "x", "frequency_penalty": 0, "logprobs": False, "n": 1, "echo": False, "tools": []}, "text")


@pytest.mark.parametrize("body,endpoint,param", [
    ([], "text", None), ({"prompt": ""}, "text", "prompt"), ({"prompt": 3}, "text", "prompt"), ({"messages": []}, "chat", "messages"),
    ({"messages": [{"role": "user"}]}, "chat", "messages"), ({"prompt": "x", "n": 2}, "text", "n"), ({"prompt": "x", "stop": ["a"]}, "text", "stop"),
    ({"prompt": "x", "stream": "yes"}, "text", "stream"), ({"prompt": "x", "max_tokens": 0}, "text", "max_tokens"),
    ({"prompt": "x", "max_tokens": 1.5}, "text", "max_tokens"), ({"prompt": "x", "seed": "1"}, "text", "seed"),
    ({"prompt": "x", "cache_key": ""}, "text", "cache_key"), ({"prompt": "x", "temperature": 0.5}, "text", "temperature"),
    ({"prompt": "x", "presence_penalty": 0.5}, "text", "presence_penalty"), ({"prompt": "x", "logprobs": True}, "text", "logprobs"),
    ({"prompt": "x", "tools": [{"type": "function"}]}, "text", "tools"), ({"prompt": "x", "stream_options": {"include_usage": True}}, "text", "stream_options"),
    ({"prompt": "x", "stream": True, "stream_options": {"foo": 1}}, "text", "stream_options.foo"),
    ({"prompt": "x", "stream": True, "stream_options": {"include_usage": "y"}}, "text", "stream_options.include_usage"),
])
def test_translation_refuses_what_the_engine_cannot_do(body, endpoint, param):
    with pytest.raises(ApiError) as info:
        to_bridge_request(body, endpoint)
    assert info.value.param == param and info.value.status == 400 and info.value.body()["error"]["param"] == param


def test_reply_shapes_and_finish_reason():
    c = to_openai_reply("text", RESULT, "m", 3, "id1")
    assert c["id"] == "cmpl-id1" and c["object"] == "text_completion" and c["choices"][0]["text"] == "abc" and c["choices"][0]["finish_reason"] == "length"
    assert c["usage"] == {"prompt_tokens": 4, "completion_tokens": 3, "total_tokens": 7} and c["nexrt_metrics"]["cache"] == "hit"
    ch = to_openai_reply("chat", dict(RESULT, stop_reason="eos"), "m", 10, "id2")
    assert ch["object"] == "chat.completion" and ch["choices"][0]["message"] == {"role": "assistant", "content": "abc"} and ch["choices"][0]["finish_reason"] == "stop"
    assert finish_reason({"tokens": [1], "stop_reason": None}, 1) == "length" and finish_reason({"tokens": [1], "stop_reason": None}, 5) == "stop"
    assert wants_usage_chunk({"stream": True, "stream_options": {"include_usage": True}}) and not wants_usage_chunk({})
    for bad, status in (("x", 502), ({"error": "bad request: nope"}, 400), ({"error": "RequestResetError"}, 502), (dict(RESULT, status=3), 502), ({"status": 0}, 502)):
        with pytest.raises(ApiError) as info:
            check_bridge_result(bad)
        assert info.value.status == status


def _parse_sse(chunks):
    out = []
    for c in chunks:
        assert c.startswith("data: ") and c.endswith("\n\n")
        body = c[6:-2]
        out.append(body if body == "[DONE]" else json.loads(body))
    return out


def test_sse_stream_for_chat_and_text():
    events = [{"type": "delta", "text": "ab"}, {"type": "delta", "text": "c"}, dict(RESULT, type="done")]
    chat = _parse_sse(sse_events("chat", iter(events), "m", 3, True, "r"))
    assert chat[0]["choices"][0]["delta"] == {"role": "assistant"} and chat[0]["usage"] is None
    assert [c["choices"][0]["delta"].get("content") for c in chat[1:3]] == ["ab", "c"]
    assert chat[3]["choices"][0]["finish_reason"] == "length" and chat[4]["choices"] == [] and chat[4]["usage"]["total_tokens"] == 7 and chat[5] == "[DONE]"
    text = _parse_sse(sse_events("text", iter(events), "m", 3, False, "r"))
    assert [c["choices"][0]["text"] for c in text[:2]] == ["ab", "c"] and "usage" not in text[0] and text[-1] == "[DONE]" and len(text) == 4
    err = _parse_sse(sse_events("text", iter([{"type": "error", "error": "boom"}]), "m", 3, False))
    assert err[0]["error"]["message"] == "boom" and err[1] == "[DONE]"
    early = _parse_sse(sse_events("text", iter([{"type": "delta", "text": "a"}]), "m", 3, False))
    assert "ended early" in early[1]["error"]["message"]


@pytest.fixture()
def facade():
    calls = []

    def call(req, host, port, timeout):
        calls.append(req)
        if req.get("text") == "explode":
            raise ConnectionRefusedError("down")
        return dict(RESULT)

    def stream(req, host, port, timeout):
        # a generator, like bridge_client.stream_request: it connects when first advanced
        calls.append(req)
        if req.get("text") == "explode":
            raise ConnectionRefusedError("down")
        yield {"type": "delta", "text": "abc"}
        if req.get("text") == "dies":
            raise ConnectionResetError("backend went away")
        yield dict(RESULT, type="done")

    state = FacadeState(model_name="m", call=call, stream=stream, queue_timeout=0.2)
    srv = OpenAIServer(("127.0.0.1", 0), state)
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    yield srv.server_address[1], calls, state
    srv.shutdown()
    srv.server_close()


def _http(port, method, path, body=None):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=10)
    c.request(method, path, body=None if body is None else json.dumps(body), headers={"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read().decode()
    c.close()
    return r.status, data


def test_http_round_trip(facade):
    port, calls, state = facade
    assert json.loads(_http(port, "GET", "/health")[1])["status"] == "ok"
    assert json.loads(_http(port, "GET", "/v1/models")[1])["data"][0]["id"] == "m"
    assert _http(port, "GET", "/v1/models/m")[0] == 200 and _http(port, "GET", "/v1/models/zzz")[0] == 404 and _http(port, "GET", "/nope")[0] == 404
    status, data = _http(port, "POST", "/v1/completions", {"model": "m", "prompt": "hi", "max_tokens": 3})
    assert status == 200 and json.loads(data)["choices"][0]["text"] == "abc" and calls[-1] == {"max_new": 3, "text": "hi"}
    status, data = _http(port, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "q"}], "stream": True, "stream_options": {"include_usage": True}})
    assert status == 200 and data.strip().endswith("data: [DONE]") and '"content": "abc"' in data and '"total_tokens": 7' in data
    assert _http(port, "POST", "/v1/completions", {"prompt": "hi", "n": 3})[0] == 400
    assert _http(port, "POST", "/v1/completions", {"model": "other", "prompt": "hi"})[0] == 404
    assert _http(port, "POST", "/v1/embeddings", {"input": "x"})[0] == 404
    assert _http(port, "POST", "/v1/completions", {"prompt": "explode"})[0] == 502
    # a stream whose backend is unreachable is a 502 JSON reply, not a 200 with a broken body
    status, data = _http(port, "POST", "/v1/completions", {"prompt": "explode", "stream": True})
    assert status == 502 and json.loads(data)["error"]["type"] == "backend_error"
    # a backend that dies in mid-stream: the delta, an in-band error, and the stream still ends with [DONE]
    status, data = _http(port, "POST", "/v1/completions", {"prompt": "dies", "stream": True})
    assert status == 200 and '"text": "abc"' in data and "backend went away" in data and data.strip().endswith("data: [DONE]")
    # one slot: while it is held a second request is refused after the queue timeout
    state.slot.acquire()
    try:
        assert _http(port, "POST", "/v1/completions", {"prompt": "hi"})[0] == 429
    finally:
        state.slot.release()
    assert _http(port, "POST", "/v1/completions", {"prompt": "hi"})[0] == 200


@pytest.mark.parametrize("body", ["[]", '"text"', "5", "null", "true"])
def test_non_object_body_is_a_400_and_never_reaches_the_backend(facade, body):
    port, calls, _ = facade
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=10)
    c.request("POST", "/v1/chat/completions", body=body, headers={"Content-Type": "application/json"})
    r = c.getresponse()
    data = json.loads(r.read().decode())
    c.close()
    assert r.status == 400 and data["error"]["type"] == "invalid_request_error" and calls == []


def test_backend_device_status_is_an_error_in_json_and_in_the_stream():
    """A reply whose device status word is not zero is never presented as a completion (reference
    tests/test_openai_serve.py: test_json_and_sse_surface_nonzero_backend_status_as_errors)."""
    bad = dict(RESULT, status=3)
    state = FacadeState(model_name="m", call=lambda *a: dict(bad), stream=lambda *a: iter([{"type": "delta", "text": "ab"}, dict(bad, type="done")]))
    srv = OpenAIServer(("127.0.0.1", 0), state)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        port = srv.server_address[1]
        status, data = _http(port, "POST", "/v1/completions", {"prompt": "hi"})
        assert status == 502 and "device status 3" in json.loads(data)["error"]["message"]
        status, data = _http(port, "POST", "/v1/completions", {"prompt": "hi", "stream": True})
        chunks = [json.loads(l[6:]) for l in data.splitlines() if l.startswith("data: {")]
        assert status == 200 and data.strip().endswith("data: [DONE]")
        assert any("error" in c for c in chunks) and not any(c.get("choices") and c["choices"][0].get("finish_reason") for c in chunks if "choices" in c)
    finally:
        srv.shutdown()
        srv.server_close()


def test_a_stalled_stream_reader_gives_the_engine_slot_back():
    """The slot is held while a stream runs.  A client that connects, asks for a stream and then reads nothing must lose it
    after the write timeout, the backend stream must be closed, and the next request must be served (reference
    tests/test_openai_serve.py: test_stalled_sse_reader_releases_backend_lock_for_next_request)."""
    import socket
    import time

    closed = threading.Event()

    def stream(req, host, port, timeout):
        try:
            for _ in range(1 << 20):
                yield {"type": "delta", "text": "x" * 65536}
        finally:
            closed.set()

    state = FacadeState(model_name="m", call=lambda *a: dict(RESULT), stream=stream, queue_timeout=5.0, write_timeout=0.3)
    srv = OpenAIServer(("127.0.0.1", 0), state)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    s = socket.create_connection(("127.0.0.1", srv.server_address[1]))
    try:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_RCVBUF, 4096)
        body = json.dumps({"prompt": "hi", "stream": True}).encode()
        s.sendall(b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: " + str(len(body)).encode() + b"\r\n\r\n" + body)
        t0 = time.monotonic()
        assert closed.wait(20.0), "the stalled stream was never given up"
        status, data = _http(srv.server_address[1], "POST", "/v1/completions", {"prompt": "hi"})
        assert status == 200 and json.loads(data)["choices"][0]["text"] == "abc" and time.monotonic() - t0 < 25.0
    finally:
        s.close()
        srv.shutdown()
        srv.server_close()


def test_translation_and_reply_checks_survive_arbitrary_json():
    """Random request bodies and random backend replies: the facade answers with ``ApiError`` (400 / 502) or a valid
    object, never with another exception."""
    import random

    rng = random.Random(2)

    def value(depth=0):
        c = rng.randrange(13)
        if c == 0:
            return None
        if c == 1:
            return rng.choice([True, False])
        if c == 2:
            return rng.choice([0, 1, -1, 5, 1 << 70])
        if c == 3:
            return rng.choice([0.0, 1.5, float("nan"), -2.0])
        if c == 4:
            return rng.choice(["", "a", "héllo"])
        if c == 5 and depth < 2:
            return [value(depth + 1) for _ in range(rng.randrange(4))]
        if c == 6 and depth < 2:
            return {rng.choice(["role", "content", "include_usage", "type", "x"]): value(depth + 1) for _ in range(rng.randrange(3))}
        if c == 7:
            return [{"role": "user", "content": "hi"}]
        return rng.choice(["a", 3, 0.5])

    keys = ["model", "prompt", "messages", "max_tokens", "max_completion_tokens", "stream", "stream_options", "n", "stop", "seed", "cache_key", "temperature",
            "top_p", "top_k", "tools", "tool_choice", "logprobs", "logit_bias", "presence_penalty", "frequency_penalty", "response_format", "user", "echo"]
    ok = 0
    for _ in range(3000):
        body = value() if rng.random() < 0.05 else {k: value() for k in rng.sample(keys, rng.randrange(0, 5))}
        if isinstance(body, dict) and rng.random() < 0.6:
            body.setdefault(*rng.choice([("prompt", "hello"), ("messages", [{"role": "user", "content": "x"}])]))
        for endpoint in ("chat", "text"):
            try:
                json.dumps(to_bridge_request(body, endpoint, forward_sampling=rng.random() < 0.5))
                ok += 1
            except ApiError as error:
                assert error.status in (400, 404)
    assert ok > 50
    fields = ["tokens", "generated_text", "status", "stop_reason", "prompt_tokens", "error", "cache"]
    for _ in range(3000):
        res = value() if rng.random() < 0.2 else {k: value() for k in rng.sample(fields, rng.randrange(0, 6))}
        try:
            to_openai_reply(rng.choice(["chat", "text"]), check_bridge_result(res), "m", 5)
        except ApiError as error:
            assert error.status in (400, 502)
        events = [res if isinstance(res, dict) else {"type": "delta", "text": "a"}, {"type": "done", "tokens": [1], "status": 0}]
        assert list(sse_events("chat", iter(events), "m", 5, True))[-1] == "data: [DONE]\n\n"
