"""Interactive streaming chat against the OpenAI-compatible facade.

Keeps the whole conversation as one growing prompt and sends it with a stable ``cache_key``, so each
turn is served as an APPEND of the retained prompt boundary (same idea as the reference's
``tools/stream_chat.py:56-116``).  ``/reset`` starts a new conversation, ``/quit`` leaves.

    python -m nexrt_b200.serve.stream_chat --url http://127.0.0.1:8000/v1
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import urllib.error
import urllib.request
import uuid
from typing import Iterator, List, Optional


def completion_url(base: str) -> str:
    base = base.rstrip("/")
    return base if base.endswith("/chat/completions") else base + "/chat/completions"


def payload(model: str, messages: List[dict], cache_key: str, max_tokens: int, seed: Optional[int] = None) -> dict:
    body = {"model": model, "messages": messages, "max_tokens": max_tokens, "stream": True, "cache_key": cache_key}
    if seed is not None:
        body["seed"] = seed
    return body


def parse_sse(lines: Iterator[bytes]) -> Iterator[dict]:
    """Yield the JSON objects of an SSE stream until ``[DONE]``."""
    for raw in lines:
        line = raw.decode("utf-8").strip()
        if not line.startswith("data:"):
            continue
        data = line[5:].strip()
        if data == "[DONE]":
            return
        yield json.loads(data)


def stream_reply(url: str, body: dict, api_key: str = "EMPTY", timeout: float = 1800.0, out=sys.stdout) -> str:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json", "Authorization": f"Bearer {api_key}"})
    text = []
    with urllib.request.urlopen(req, timeout=timeout) as resp:
        for ev in parse_sse(resp):
            if "error" in ev:
                raise RuntimeError(ev["error"].get("message", str(ev["error"])))
            for choice in ev.get("choices", ()):
                piece = choice.get("delta", {}).get("content")
                if piece:
                    text.append(piece)
                    out.write(piece)
                    out.flush()
    out.write("\n")
    return "".join(text)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Interactive streaming chat")
    ap.add_argument("--url", default="http://127.0.0.1:8000/v1")
    ap.add_argument("--model", default="Nex-N2.5-Pro")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--system", default=None)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--api-key", default=os.environ.get("OPENAI_API_KEY", "EMPTY"))
    a = ap.parse_args(argv)
    url = completion_url(a.url)

    def fresh():
        return ([{"role": "system", "content": a.system}] if a.system else []), uuid.uuid4().hex

    messages, key = fresh()
    while True:
        try:
            line = input("> ").strip()
        except (EOFError, KeyboardInterrupt):
            print()
            return 0
        if not line:
            continue
        if line == "/quit":
            return 0
        if line == "/reset":
            messages, key = fresh()
            continue
        messages.append({"role": "user", "content": line})
        try:
            reply = stream_reply(url, payload(a.model, messages, key, a.max_tokens, a.seed), a.api_key)
            messages.append({"role": "assistant", "content": reply})
        except (urllib.error.URLError, RuntimeError, OSError) as error:
            print(f"[error] {error}")
            messages.pop()


if __name__ == "__main__":
    raise SystemExit(main())
