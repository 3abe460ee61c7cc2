"""Operator entry points: ``preflight`` (read-only checks), ``serve`` (workers + OpenAI facade under one
parent) and ``smoke`` (one request through the running server).  Replaces the reference's shell
scripts (preflight / serve / smoke under ``sglang_prefill/``) with one module so the same checks run in
tests.

    python -m nexrt_b200.serve.launch preflight --tp 8
    python -m nexrt_b200.serve.launch serve --tp 8 --mode bs1 --port 9411 --http-port 8000
    python -m nexrt_b200.serve.launch smoke --port 9411
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import signal
import subprocess
import sys
import time
from pathlib import Path
from typing import Dict, List


def preflight(tp: int, layers_dir=None, probe_gpu: bool = True, mode: str = "bs1", n_layers: int = 0) -> List[Dict]:
    """Return ``[{check, ok, detail}]``.  Reads state only: nothing on the GPUs is changed.  ``n_layers`` (0 = the full
    model) is how many ``layer.<L>`` files the directory must hold; ``mode`` adds the draft weights of a speculative mode
    (their absence is reported but is not a failure: the server then runs a random draft)."""
    out: List[Dict] = []

    def add(check, ok, detail=""):
        out.append({"check": check, "ok": bool(ok), "detail": str(detail)})

    add("tp degree", tp in (1, 2, 4, 8), tp)
    add("nvcc on PATH", shutil.which("nvcc") is not None, shutil.which("nvcc") or "missing (needed only to rebuild the kernels)")
    lib = Path(__file__).resolve().parents[1] / "libnexrt_b200.so"
    add("kernel library built", lib.is_file(), lib)
    if layers_dir:
        d = Path(layers_dir)
        if not n_layers:
            from ..config import full_config

            n_layers = full_config().n_layers
        need = ["embed_tokens.safetensors", "norm.safetensors", "lm_head.safetensors"] + [f"layer.{l}.safetensors" for l in range(n_layers)]
        missing = [n for n in need if not (d / n).is_file()]
        add("layer directory", not missing, f"missing {missing[:4]}{' ...' if len(missing) > 4 else ''} ({len(missing)} of {len(need)} files)" if missing else d)
        if mode == "mtp":
            have = (d / "mtp.safetensors").is_file()
            add("MTP draft weights", True, d / "mtp.safetensors" if have else "mtp.safetensors not found: the server will run a RANDOM draft (acceptance ~1)")
    if mode == "dflash":
        from ..dflash.config import DFLASH_CONFIG, DFLASH_WEIGHTS

        have = DFLASH_CONFIG.is_file() and DFLASH_WEIGHTS.is_file()
        add("DFlash draft weights", True, DFLASH_WEIGHTS if have else f"{DFLASH_CONFIG} / {DFLASH_WEIGHTS} not found (NEXRT_DFLASH_DIR): the server will run a RANDOM draft")
    if probe_gpu:
        try:
            import torch

            n = torch.cuda.device_count()
            add("visible GPUs", n >= tp, f"{n} visible, {tp} needed")
            if n >= 1:
                cc = torch.cuda.get_device_capability(0)
                add("compute capability 10.x", cc[0] == 10, f"sm_{cc[0]}{cc[1]}")
                add("peer access", all(torch.cuda.can_device_access_peer(0, j) for j in range(1, min(n, tp))), "GPU 0 -> peers")
        except Exception as error:  # noqa: BLE001
            add("torch / CUDA import", False, error)
    return out


def serve(a) -> int:
    """Start ``tp`` workers under torchrun and the HTTP facade; stop both on SIGINT / SIGTERM or when
    either exits."""
    worker = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nproc-per-node", str(a.tp),
              "-m", "nexrt_b200.serve.bridge_serve", "--listen", str(a.port), "--mode", a.mode, "--context", str(a.context)]
    if a.layers:
        worker += ["--layers", str(a.layers)]
    if a.layers_dir:
        worker += ["--layers-dir", a.layers_dir]
    if a.tokenizer:
        worker += ["--tokenizer", a.tokenizer]
    if a.cp:
        worker += ["--cp"]
    if a.wide_prefill:
        worker += ["--wide-prefill", str(a.wide_prefill)]
    facade = [sys.executable, "-m", "nexrt_b200.serve.openai_serve", "--port", str(a.http_port), "--backend-port", str(a.port), "--model-name", a.model_name]
    if a.forward_sampling:
        facade += ["--forward-sampling"]
    procs = [subprocess.Popen(worker, start_new_session=True), subprocess.Popen(facade, start_new_session=True)]
    stop = []
    for sig in (signal.SIGINT, signal.SIGTERM):
        signal.signal(sig, lambda *_: stop.append(1))
    try:
        while not stop and all(p.poll() is None for p in procs):
            time.sleep(0.5)
    finally:
        for p in procs:                      # each child leads its own process group: signal exactly that group
            if p.poll() is None:
                os.killpg(p.pid, signal.SIGTERM)
        for p in procs:
            try:
                p.wait(30)
            except subprocess.TimeoutExpired:
                os.killpg(p.pid, signal.SIGKILL)
    return max((p.returncode or 0) for p in procs)


def smoke(a) -> int:
    from .bridge_client import send_request

    r = send_request({"text": a.text, "max_new": a.max_new, "temperature": 0.0}, a.host, a.port, timeout=a.timeout)
    print(json.dumps({k: r.get(k) for k in ("error", "status", "stop_reason", "prompt_tokens", "ttft_s", "decode_us_per_tok", "cache", "tokens")}))
    return 0 if "error" not in r and r.get("status") == 0 and len(r.get("tokens", ())) >= 1 else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("preflight")
    p.add_argument("--tp", type=int, default=8)
    p.add_argument("--layers-dir", default=None)
    p.add_argument("--mode", default="bs1", choices=["bs1", "mtp", "dflash"])
    p.add_argument("--layers", type=int, default=0, help="layer files the directory must hold (0 = the full model)")
    s = sub.add_parser("serve")
    s.add_argument("--tp", type=int, default=8)
    s.add_argument("--mode", default="bs1", choices=["bs1", "mtp", "dflash"])
    s.add_argument("--port", type=int, default=9411)
    s.add_argument("--http-port", type=int, default=8000)
    s.add_argument("--layers", type=int, default=0)
    s.add_argument("--layers-dir", default=None)
    s.add_argument("--tokenizer", default=None)
    s.add_argument("--context", type=int, default=32768)
    s.add_argument("--cp", action="store_true")
    s.add_argument("--wide-prefill", type=int, default=0, help="rows per wide prefill chunk of the workers (0 = 8-row steps)")
    s.add_argument("--model-name", default="Nex-N2.5-Pro")
    s.add_argument("--forward-sampling", action="store_true")
    k = sub.add_parser("smoke")
    k.add_argument("--host", default="127.0.0.1")
    k.add_argument("--port", type=int, default=9411)
    k.add_argument("--text", default="The capital of France is")
    k.add_argument("--max-new", type=int, default=16)
    k.add_argument("--timeout", type=float, default=600.0)
    a = ap.parse_args(argv)
    if a.cmd == "preflight":
        rows = preflight(a.tp, a.layers_dir, mode=a.mode, n_layers=a.layers)
        for r in rows:
            print(f"[{'ok' if r['ok'] else 'FAIL'}] {r['check']}: {r['detail']}")
        return 0 if all(r["ok"] for r in rows) else 1
    return serve(a) if a.cmd == "serve" else smoke(a)


if __name__ == "__main__":
    raise SystemExit(main())
