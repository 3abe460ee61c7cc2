"""Minimal client of the bridge socket: one JSON line out, one JSON object (or an NDJSON stream) back.

Counterpart of the reference's ``sglang_prefill/bridge_client.py`` (``BRIDGE.md:28-56``).

    python -m nexrt_b200.serve.bridge_client --port 9411 --text "hello" --max-new 64 --stream
    python -m nexrt_b200.serve.bridge_client --port 9411 --file prompt.txt --chat

A prompt file is read HERE (UTF-8) and travels as inline ``text``: the server takes no paths from the socket, and a file
that cannot be read ends the client (exit code 2) before it connects.
"""

from __future__ import annotations

import argparse
import json
import socket
import sys
from typing import Dict, Iterator, Optional


def _connect(host: str, port: int, timeout: Optional[float]):
    s = socket.create_connection((host, port), timeout=timeout)
    return s


def send_request(request: Dict, host: str = "127.0.0.1", port: int = 9411, timeout: Optional[float] = 600.0) -> Dict:
    """Send one non-streaming request and return the decoded reply."""
    with _connect(host, port, timeout) as s:
        s.sendall((json.dumps(request) + "\n").encode())
        buf = b""
        while not buf.endswith(b"\n"):
            part = s.recv(1 << 16)
            if not part:
                break
            buf += part
    if not buf:
        raise ConnectionError("the server closed the connection without a reply")
    return json.loads(buf.decode("utf-8"))


def stream_request(request: Dict, host: str = "127.0.0.1", port: int = 9411, timeout: Optional[float] = 600.0) -> Iterator[Dict]:
    """Send a streaming request; yields every NDJSON event (``delta`` events, then ``final`` or ``error``)."""
    req = dict(request, stream=True)
    with _connect(host, port, timeout) as s:
        s.sendall((json.dumps(req) + "\n").encode())
        with s.makefile("rb") as f:
            for line in f:
                line = line.strip()
                if line:
                    yield json.loads(line.decode("utf-8"))


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="nexrt_b200 bridge client")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=9411)
    p.add_argument("--text")
    p.add_argument("--file", help="UTF-8 prompt file, read by the client and sent as inline text")
    p.add_argument("--ids", help="comma separated token ids")
    p.add_argument("--chat", action="store_true")
    p.add_argument("--max-new", type=int, default=128)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--cache-key")
    p.add_argument("--temperature", type=float)
    p.add_argument("--top-p", type=float)
    p.add_argument("--top-k", type=int)
    p.add_argument("--stream", action="store_true")
    p.add_argument("--shutdown", action="store_true")
    a = p.parse_args(argv)
    if sum(v is not None for v in (a.text, a.file, a.ids)) > 1:
        p.error("give one of --text, --file, --ids")
    if a.file is not None:
        try:
            with open(a.file, "r", encoding="utf-8") as fh:
                a.text = fh.read()
        except (OSError, UnicodeDecodeError) as error:
            p.error(f"cannot read {a.file}: {error}")          # exits with code 2, nothing was sent
    if a.shutdown:
        print(json.dumps(send_request({"cmd": "shutdown"}, a.host, a.port)))
        return 0
    req: Dict = {"max_new": a.max_new, "seed": a.seed}
    if a.ids:
        req["ids"] = [int(t) for t in a.ids.split(",")]
    else:
        req["text"] = a.text if a.text is not None else sys.stdin.read()
        if a.chat:
            req["chat"] = True
    for key, val in (("cache_key", a.cache_key), ("temperature", a.temperature), ("top_p", a.top_p), ("top_k", a.top_k)):
        if val is not None:
            req[key] = val
    if a.stream:
        for ev in stream_request(req, a.host, a.port):
            if ev.get("type") == "delta":
                sys.stdout.write(ev.get("text", ""))
                sys.stdout.flush()
            else:
                print("\n" + json.dumps(ev))
    else:
        print(json.dumps(send_request(req, a.host, a.port), ensure_ascii=False))
    return 0


if __name__ == "__main__":
    sys.exit(main())
