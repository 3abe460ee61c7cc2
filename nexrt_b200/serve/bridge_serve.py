"""The serving worker: one process per GPU, rank 0 owns a TCP JSON-line socket, every request runs
in tensor-parallel lock-step.

Shape of the reference's ``bridge_serve.worker`` (``nex_n2_5_pro/sglang_prefill/bridge_serve.py:
173-1605``; protocol ``BRIDGE.md:28-56``): rank 0 accepts one JSON line per connection, validates
and tokenises it, broadcasts the request to the other ranks, all ranks run the same pipeline

    cache plan + TP consensus -> lease (PREFILL | APPEND | HIT) -> chunked prefill -> boundary
    consensus -> decode (1-batch, MTP or DFlash; tokens stream to the client from rank 0) ->
    restore the prompt boundary -> retain consensus,

and rank 0 answers with one JSON object (or an NDJSON stream).  Idle ranks park in the request
broadcast; rank 0's ``accept`` times out every 60 s and broadcasts a heartbeat so the process-group
watchdog never fires.  ``{"cmd":"shutdown"}`` stops the server.  Failures follow
``serve_control``: collective reset or terminate all ranks with exit code 2.

Differences: prefill is the engine's own (no SGLang process state to keep in step), the decode
back end is behind a small interface so the whole request pipeline runs against a fake back end on
CPU, and host-side control traffic uses a gloo group (``broadcast_object_list``) instead of NCCL.
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import sys
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from ..sampling import DEFAULT_SAMPLING, checked_sampling_config, resolve_sampling_config, sampling_defaults
from .bridge import PrefillSession, chunked_prefill
from .cache_consensus import (all_gather_records, boundary_record, request_fingerprint, request_record, resolve_boundary,
                              resolve_request, resolve_retain, retain_record)
from .cache_lifecycle import CacheBoundary, CacheDecision, CachedSession, CachePhase
from .serve_control import (RequestResetError, cache_key_for_request, dispatch_port_request, execute_request_with_consensus,
                            reset_failed_request)
from .stream_protocol import BridgeStreamWriter, decode_visible_text

HEARTBEAT_S = 60.0
DEFAULT_PORT = 9411
MAX_NEW_LIMIT = 1 << 16


# ---- tokenizers ------------------------------------------------------------------------------------
class ByteTokenizer:
    """UTF-8 bytes as token ids (offset 3; 0 = pad, 1 = bos, 2 = eos).  Used when no tokenizer
    directory is given (synthetic weights, tests)."""

    eos_token_id = 2

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        return [b + 3 for b in text.encode("utf-8")]

    def decode(self, ids, skip_special_tokens: bool = False, clean_up_tokenization_spaces: bool = False) -> str:
        return bytes((int(i) - 3) & 0xFF for i in ids if int(i) >= 3).decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True):
        text = "".join(f"<{m['role']}>{m['content']}\n" for m in messages) + ("<assistant>" if add_generation_prompt else "")
        return self.encode(text) if tokenize else text


def load_tokenizer(path: Optional[str]):
    if not path:
        return ByteTokenizer()
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(path)


# ---- stop tokens --------------------------------------------------------------------------------------------
# a turn also ends where the model opens a tool call: the client, not the server, continues from there
TOOL_CALL_OPENERS = ("<tool_call>", "<|tool_call_begin|>", "<|tool_calls_begin|>", "<function_call>", "<|action_start|>")


def resolve_stop_ids(tokenizer, model_dir: Optional[str] = None, openers: Sequence[str] = TOOL_CALL_OPENERS) -> Tuple[int, ...]:
    """Every token id that ends a generation, sorted: the tokenizer's ``eos_token_id`` (one id or a list), the
    ``eos_token_id`` of ``generation_config.json`` in ``model_dir`` (one id, a list, null or no file), and the ids of the
    tool-call opener strings the tokenizer knows as single tokens (an id equal to ``unk_token_id``, negative or missing
    means it does not).  Same sources as the reference's server (sglang_prefill/bridge_serve.py:140-165)."""
    def as_ids(value) -> List[int]:
        if value is None or isinstance(value, bool):
            return []
        if isinstance(value, int):
            return [value]
        return [int(v) for v in value if v is not None and not isinstance(v, bool)]

    ids = set(as_ids(getattr(tokenizer, "eos_token_id", None)))
    if model_dir:
        path = os.path.join(model_dir, "generation_config.json")
        if os.path.isfile(path):
            try:
                with open(path, "r", encoding="utf-8") as fh:
                    ids.update(as_ids(json.load(fh).get("eos_token_id")))
            except (OSError, ValueError, AttributeError, TypeError):
                pass        # an unreadable generation config adds no stop ids; the tokenizer's still hold
    convert = getattr(tokenizer, "convert_tokens_to_ids", None)
    unk = getattr(tokenizer, "unk_token_id", None)
    if callable(convert):
        for text in openers:
            try:
                tid = convert(text)
            except Exception:  # noqa: BLE001 - tokenizers differ in what they raise for an unknown string
                tid = None
            if isinstance(tid, int) and not isinstance(tid, bool) and tid >= 0 and tid != unk:
                ids.add(tid)
    return tuple(sorted(i for i in ids if i >= 0))


# ---- request validation -------------------------------------------------------------------------------
class BadRequest(ValueError):
    pass


def validate_request(req: Dict, capacity: int, mode: str, defaults=DEFAULT_SAMPLING) -> Dict:
    """Normalise one client request or raise :class:`BadRequest` (rank 0, before any broadcast)."""
    if not isinstance(req, dict):
        raise BadRequest("request must be a JSON object")
    if req.get("cmd") == "shutdown":
        return {"cmd": "shutdown"}
    known = {"text", "ids", "chat", "messages", "max_new", "seed", "cache_key", "temperature", "top_p", "top_k", "stream", "cmd"}
    unknown = set(req) - known
    if unknown:
        raise BadRequest(f"unknown fields: {sorted(unknown)}")
    if ("text" in req) + ("ids" in req) + ("messages" in req) != 1:
        raise BadRequest("exactly one of text, ids, messages is required")
    if "text" in req and not isinstance(req["text"], str):
        raise BadRequest("text must be a string")
    if "ids" in req and not (isinstance(req["ids"], list) and req["ids"] and all(isinstance(t, int) and not isinstance(t, bool) and t >= 0 for t in req["ids"])):
        raise BadRequest("ids must be a non-empty list of non-negative integers")
    if "messages" in req:
        msgs = req["messages"]
        if not (isinstance(msgs, list) and msgs and all(isinstance(m, dict) and isinstance(m.get("role"), str) and isinstance(m.get("content"), str)
                                                        for m in msgs)):
            raise BadRequest("messages must be a non-empty list of {role: string, content: string}")
    for flag in ("chat", "stream"):
        if flag in req and not isinstance(req[flag], bool):
            raise BadRequest(f"{flag} must be a boolean")
    max_new = req.get("max_new", 128)
    if isinstance(max_new, bool) or not isinstance(max_new, int) or not 1 <= max_new <= MAX_NEW_LIMIT:
        raise BadRequest(f"max_new must be an integer in [1, {MAX_NEW_LIMIT}]")
    seed = req.get("seed", 0)
    if isinstance(seed, bool) or not isinstance(seed, int) or not 0 <= seed < (1 << 64):
        raise BadRequest("seed must be an unsigned 64-bit integer")
    speculative = mode != "bs1"
    if speculative and "top_k" in req:
        raise BadRequest("top_k can be set in 1-batch mode only")
    try:
        t, p, k = resolve_sampling_config(defaults, req.get("temperature"), req.get("top_p"), req.get("top_k"))
        key = cache_key_for_request(req.get("cache_key"), speculative=speculative)
    except ValueError as error:
        raise BadRequest(str(error)) from error
    if key is not None and not (isinstance(key, str) and key):
        raise BadRequest("cache_key must be a non-empty string")
    return {"text": req.get("text"), "ids": req.get("ids"), "messages": req.get("messages"), "chat": bool(req.get("chat", False)),
            "max_new": max_new, "seed": seed, "cache_key": key, "temperature": t, "top_p": p, "top_k": k, "stream": bool(req.get("stream", False)),
            "capacity": capacity}


# ---- decode back ends ------------------------------------------------------------------------------------
class EngineBackend:
    """The real back end: a :class:`DecodeEngine` plus, by mode, an MTP draft or a DFlash block."""

    def __init__(self, engine, mode: str = "bs1", spec_block=None, chunk: int = 8, model_epoch: str = "random-init"):
        self.eng, self.mode, self.block, self.chunk = engine, mode, spec_block, chunk
        self.capacity = engine._kv_budget()
        self.model_epoch = model_epoch
        self.vocab = engine.cfg.vocab

    def set_sampling(self, seed, t, p, k) -> None:
        self.eng.head.set_sampling_config(seed, t, p, k)

    def prefill(self, tokens: Sequence[int], resume: Optional[PrefillSession], on_chunk) -> PrefillSession:
        if self.mode == "mtp":
            first = self.block.prefill(tokens, chunk=self.chunk)
            on_chunk(0, len(tokens))
            return PrefillSession(tuple(tokens), first, self.eng._snapshot())
        if self.mode == "dflash":
            first = self.block.prefill(tokens)
            on_chunk(0, len(tokens))
            return PrefillSession(tuple(tokens), first, self.eng._snapshot())
        _, session = chunked_prefill(self.eng, tokens, self.chunk, on_chunk=lambda s, e, nt: on_chunk(s, e) if e > s else None,
                                     resume=resume, return_session=True)
        return session

    def boundary(self) -> CacheBoundary:
        d = self.eng.read_ctl()
        return CacheBoundary(d["committed_len"], d["pending"], 0)

    def restore(self, session: PrefillSession) -> CacheBoundary:
        self.eng._restore(session.snapshot)
        return self.boundary()

    def decode(self, max_new: int, eos_ids, on_tokens) -> Dict:
        eos = tuple(eos_ids or ())          # every stop id ends the request, not only the first
        stats: Dict = {}
        if self.mode == "mtp":
            from ..mtp import generate_mtp

            toks = generate_mtp(self.block, max_new=max_new, eos=eos, on_tokens=on_tokens, stats=stats)
        elif self.mode == "dflash":
            from ..dflash import generate_dflash

            toks = generate_dflash(self.block, max_new=max_new, eos=eos, on_tokens=on_tokens, stats=stats)
        else:
            toks = self.eng.generate(max_new=max_new, eos=eos, on_tokens=on_tokens)
        return {"tokens": toks, **stats}

    def verify_tokens(self, session: PrefillSession, tokens: Sequence[int], req: Dict) -> bool:
        """Replay the request from the restored prompt boundary on the plain one-row decode path (eager, no
        graph, no drafts) and compare: speculative modes must emit exactly the plain stream."""
        self.eng._restore(session.snapshot)
        plain = [session.first_token]
        from ..runtime.control import Ctl

        for _ in range(len(tokens) - 1):
            self.eng.step(1)
            w = self.eng.read_ctl()
            if w["status"] != 0:
                return False
            plain.append(int(w["pending"]))
        return plain == list(tokens)

    def status(self) -> int:
        return self.eng.status_max()

    def reset(self, reason: str, cache, runtime_state) -> None:
        import torch

        reset_failed_request(reason, cache=cache, runtime_state=runtime_state, engine=self.eng,
                             speculative_blocks=(self.block,) if self.block is not None else (), synchronize=torch.cuda.synchronize)


@dataclass
class ServerState:
    cache: CachedSession
    session: Optional[PrefillSession] = None
    active_lease: object = None
    request_kind: int = 0


class BridgeServer:
    """Per-rank request pipeline + the rank-0 listen loop."""

    def __init__(self, backend, tokenizer, rank: int = 0, world: int = 1, control_group=None, mode: str = "bs1",
                 report_path: Optional[str] = None, gather: Optional[Callable] = None, log: Callable[[str], None] = print,
                 consensus_fault_rank: Optional[int] = None, verify: bool = False, model_dir: Optional[str] = None):
        self.backend, self.tok, self.rank, self.world, self.group, self.mode = backend, tokenizer, rank, world, control_group, mode
        self.state = ServerState(CachedSession(backend.capacity, backend.model_epoch))
        self.report_path = report_path or os.environ.get("NEXRT_SERVE_REPORT")
        self.report: List[Dict] = []
        self._gather = gather or (lambda rec: all_gather_records(rec, group=self.group))
        self.log = log if rank == 0 else (lambda *_: None)
        self.stop_ids = resolve_stop_ids(tokenizer, model_dir)
        self.sampling = sampling_defaults(model_dir)        # the model's generation_config.json over the built-in defaults
        # test-only host-side fault injection: this rank reports its READY boundary as lost on the next reuse,
        # which must turn the request into a collective PREFILL on every rank
        self.consensus_fault_rank = consensus_fault_rank
        self.verify = verify

    # ---- one request, every rank ---------------------------------------------------------------------
    def tokenize(self, req: Dict) -> List[int]:
        try:
            if req.get("ids") is not None:
                ids = list(req["ids"])
            elif req.get("messages") is not None:
                ids = list(self.tok.apply_chat_template(req["messages"], tokenize=True, add_generation_prompt=True))
            elif req.get("chat"):
                ids = list(self.tok.apply_chat_template([{"role": "user", "content": req["text"]}], tokenize=True, add_generation_prompt=True))
            else:
                ids = list(self.tok.encode(req["text"], add_special_tokens=False))
            ids = [int(t) for t in ids]
        except BadRequest:
            raise
        except Exception as error:  # noqa: BLE001 - whatever a tokenizer or its chat template raises is the request's fault, not the server's
            raise BadRequest(f"the tokenizer rejected the prompt: {type(error).__name__}: {error}") from error
        if not ids:
            raise BadRequest("empty prompt")
        if any(t < 0 or t >= self.backend.vocab for t in ids):
            raise BadRequest("token id outside the vocabulary")
        if len(ids) + req["max_new"] > self.backend.capacity:
            raise BadRequest(f"prompt of {len(ids)} tokens + max_new {req['max_new']} exceeds the context capacity {self.backend.capacity}")
        return ids

    def handle_request(self, req: Dict, ids: Sequence[int], stream: Optional[BridgeStreamWriter] = None) -> Dict:
        """The collective part of a request (identical on every rank)."""
        st, be, cache = self.state, self.backend, self.state.cache
        t0 = time.perf_counter()
        owner = req["cache_key"]
        live = be.boundary() if cache.snapshot().phase == CachePhase.READY else None
        plan = cache.plan_request(owner, ids, live_boundary=live)
        fp = request_fingerprint(owner=owner, tokens=ids, model_epoch=be.model_epoch, decode_kind=self.mode, max_new_tokens=req["max_new"],
                                 seed=req["seed"], temperature=req["temperature"], top_p=req["top_p"], top_k=req["top_k"])
        # validity 0 = "my device no longer holds the boundary I stored": turns the request into a collective PREFILL
        valid = live is None or live == cache.snapshot().boundary
        if live is not None and self.consensus_fault_rank is not None and self.rank == self.consensus_fault_rank:
            valid, self.consensus_fault_rank = False, None          # injected once
        consensus = resolve_request(self._gather(request_record(valid, plan, fp)))
        t_consensus = time.perf_counter() - t0
        lease = cache.begin_request(owner, ids, request_id=f"g{plan.generation}", live_boundary=live, force_prefill=consensus.forced_prefill)
        st.active_lease = lease
        be.set_sampling(req["seed"], req["temperature"], req["top_p"], req["top_k"])
        # ---- prefill
        t1 = time.perf_counter()
        resume = st.session if lease.decision != CacheDecision.PREFILL else None
        if lease.decision == CacheDecision.HIT:
            be.restore(st.session)
            session = st.session
        else:
            session = be.prefill(ids, resume, on_chunk=lambda s, e: cache.record_append(lease, s, e) if e > s else None)
        boundary = be.boundary()
        resolve_boundary(self._gather(boundary_record(boundary.committed_len == len(ids), lease.generation, len(ids), boundary)), "fill")
        cache.commit_fill(lease, boundary)
        st.session = session
        prefill_s = time.perf_counter() - t1
        # ---- decode
        cache.begin_decode(lease)
        emitted: List[int] = [session.first_token]
        ttft_s = time.perf_counter() - t0
        if stream is not None:
            stream.tokens([session.first_token])

        def on_tokens(toks):
            emitted.extend(toks)
            if stream is not None:
                stream.tokens(toks)

        t2 = time.perf_counter()
        stop_first = session.first_token in self.stop_ids
        stats = {"tokens": []} if (stop_first or req["max_new"] <= 1) else be.decode(req["max_new"] - 1, self.stop_ids, on_tokens)
        decode_s = time.perf_counter() - t2
        status = be.status()
        # ---- restore the prompt boundary; keep it only if every rank could
        restored = be.restore(session)
        keep, _ = resolve_retain(self._gather(retain_record(restored == boundary and status == 0 and owner is not None, lease.generation, len(ids))))
        if keep:
            cache.finish_decode(lease, restored)
        else:
            cache.abort_decode(lease, "boundary not retained")
            st.session = None
        st.active_lease = None
        toks = [session.first_token] + list(stats["tokens"])
        toks = toks[: req["max_new"]]
        verified = None
        if self.verify and hasattr(be, "verify_tokens"):
            # re-decode from the restored boundary on the plain one-row path and compare the streams
            verified = bool(be.verify_tokens(session, toks, req))
            be.restore(session)
        stop = "eos" if any(t in self.stop_ids for t in toks) else ("length" if len(toks) >= req["max_new"] else "context")
        n_dec = max(len(toks) - 1, 1)
        return {
            "tokens": toks, "generated_text": decode_visible_text(self.tok, toks, self.stop_ids), "status": status, "stop_reason": stop,
            "prompt_tokens": len(ids), "cache": lease.decision.value, "forced_prefill": consensus.forced_prefill, "mode": self.mode,
            "prefill_s": round(prefill_s, 6), "ttft_s": round(ttft_s, 6), "decode_us_per_tok": round(decode_s * 1e6 / n_dec, 2),
            "consensus_ms": round(t_consensus * 1e3, 3), "rounds": stats.get("rounds"), "accept_mean": stats.get("accept_mean"),
            "verified": verified, "cache_base_tokens": lease.base_length, "cache_retained": bool(keep),
        }

    def run_request(self, req: Dict, ids: Sequence[int], stream=None) -> Dict:
        """handle_request under the collective failure policy."""
        cache = self.state.cache

        def lifecycle():
            s = cache.snapshot()
            phase = list(CachePhase).index(s.phase)
            lease = self.state.active_lease
            return s.generation, phase, 0 if lease is None else lease.generation, self.state.request_kind

        def reset(reason: str) -> None:
            self.backend.reset(reason, cache, self.state.__dict__)
            self.state.session = None
            self.state.active_lease = None

        return execute_request_with_consensus(lambda: self.handle_request(req, ids, stream), lifecycle_state=lifecycle,
                                              gather_outcome=self._gather, reset_request=reset)

    # ---- queued requests and the cache matrix (every rank calls these with the same arguments) ------------
    def run_queue(self, requests: Sequence[Dict]) -> List[Dict]:
        """Serve a fixed list of requests in order (synthetic lengths, prompt files); a request that ends in
        a collective reset is reported and the queue goes on."""
        out = []
        for i, raw in enumerate(requests):
            req = validate_request(raw, self.backend.capacity, self.mode, self.sampling)
            ids = self.tokenize(req)
            try:
                res = self.run_request(req, ids)
            except RequestResetError as error:
                res = {"error": repr(error), "prompt_tokens": len(ids)}
            res["request"] = i
            out.append(res)
            if self.rank == 0:
                self.report.append(res)
                self.log("@@ SERVE " + json.dumps({k: v for k, v in res.items() if k not in ("tokens", "generated_text")}))
        self._flush_report()
        return out

    def cache_e2e(self, base_len: int, target_len: int, repetitions: int = 3, gen: int = 8, seed: int = 1) -> Dict:
        """PREFILL(base) -> HIT(base) -> APPEND(target) under one owner, then the same prompts without an owner
        (fresh prefills) as the oracle: a reused boundary must reproduce the oracle's tokens exactly."""
        if not 0 < base_len < target_len:
            raise ValueError("cache e2e needs 0 < base < target")
        import random

        rnd = random.Random(seed)
        target = [rnd.randrange(3, self.backend.vocab) for _ in range(target_len)]
        base = target[:base_len]
        rows, ok = [], True
        for rep in range(repetitions):
            key = f"cache-e2e-{rep}"
            steps = [("prefill", base, key), ("hit", base, key), ("append", target, key), ("oracle-base", base, None), ("oracle-target", target, None)]
            got = {}
            for name, ids, owner in steps:
                req = validate_request({"ids": ids, "max_new": gen, "temperature": 0.0, "cache_key": owner}, self.backend.capacity, self.mode, self.sampling)
                res = self.run_request(req, ids)
                got[name] = res
                rows.append({"rep": rep, "step": name, "cache": res["cache"], "prefill_s": res["prefill_s"], "ttft_s": res["ttft_s"]})
            decisions = (got["prefill"]["cache"], got["hit"]["cache"], got["append"]["cache"])
            same = got["hit"]["tokens"] == got["oracle-base"]["tokens"] == got["prefill"]["tokens"] and got["append"]["tokens"] == got["oracle-target"]["tokens"]
            ok = ok and same and decisions == ("prefill", "hit", "append")
        return {"base": base_len, "target": target_len, "repetitions": repetitions, "ok": ok, "rows": rows}

    # ---- broadcast plumbing -----------------------------------------------------------------------------
    def _broadcast(self, obj):
        if self.world == 1:
            return obj
        import torch.distributed as dist

        box = [obj]
        dist.broadcast_object_list(box, src=0, group=self.group)
        return box[0]

    def _terminate(self, error, conn) -> None:
        self.log(f"@@ SERVE fatal: {error!r}")
        if conn is not None:
            try:
                conn.sendall((json.dumps({"error": repr(error), "fatal": True}) + "\n").encode())
            except OSError:
                pass
        self._flush_report()
        os._exit(2)

    def _flush_report(self) -> None:
        if self.rank == 0 and self.report_path and self.report:
            with open(self.report_path, "a") as f:
                for r in self.report:
                    f.write(json.dumps({k: v for k, v in r.items() if k != "generated_text"}) + "\n")
            self.report.clear()

    # ---- listen loop ------------------------------------------------------------------------------------
    def serve_forever(self, host: str = "127.0.0.1", port: int = DEFAULT_PORT, ready: Optional[Callable[[int], None]] = None) -> None:
        srv = None
        if self.rank == 0:
            srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            srv.bind((host, port))
            srv.listen(8)
            srv.settimeout(HEARTBEAT_S)
            self.log(f"@@ SERVE listening on {host}:{srv.getsockname()[1]} mode={self.mode} tp={self.world}")
            if ready is not None:
                ready(srv.getsockname()[1])
        try:
            while True:
                conn, msg = None, None
                if self.rank == 0:
                    conn, msg = self._accept_one(srv)
                msg = self._broadcast(msg)
                if msg is None or msg.get("cmd") == "heartbeat":
                    continue
                if msg.get("cmd") == "shutdown":
                    if conn is not None:
                        conn.sendall(b'{"ok": true}\n')
                        conn.close()
                    break
                stream = None
                if self.rank == 0 and msg["req"]["stream"]:
                    stream = BridgeStreamWriter(conn, self.tok, self.stop_ids)
                dispatch_port_request(lambda: self.run_request(msg["req"], msg["ids"], stream), tp_rank=self.rank, conn=conn,
                                      event_stream=stream, report=self.report, terminate_fatally=self._terminate,
                                      log_reset=lambda e: self.log(f"@@ SERVE request reset: {e}"))
                self._flush_report()
        finally:
            if srv is not None:
                srv.close()

    def _accept_one(self, srv):
        """Rank 0: wait for a connection (heartbeat on timeout), read one JSON line, validate, tokenise."""
        try:
            conn, _ = srv.accept()
        except socket.timeout:
            return None, {"cmd": "heartbeat"}
        try:
            conn.settimeout(10.0)
            buf = b""
            while not buf.endswith(b"\n") and len(buf) < (64 << 20):
                part = conn.recv(1 << 16)
                if not part:
                    break
                buf += part
            req = validate_request(json.loads(buf.decode("utf-8")), self.backend.capacity, self.mode, self.sampling)
            if req.get("cmd") == "shutdown":
                return conn, req
            ids = self.tokenize(req)
            return conn, {"cmd": "request", "req": req, "ids": ids}
        except Exception as error:  # noqa: BLE001
            # nothing a client sends may take the server down: malformed JSON, a wrong field, a prompt the tokenizer refuses,
            # a socket that times out or resets - the request is answered (if the socket still takes it) and dropped
            try:
                conn.sendall((json.dumps({"error": f"bad request: {error}"}) + "\n").encode())
            except OSError:
                pass
            finally:
                conn.close()
            return None, {"cmd": "heartbeat"}


# ---- process entry point ----------------------------------------------------------------------------------
def build_backend(args, rank: int, world: int, dev, group):
    """Random-init (or checkpoint) model, engine and speculative block for this rank."""
    from ..config import full_config
    from ..decode_engine import DecodeEngine
    from ..weights import load_rank_model, random_rank_model

    cfg = full_config()
    if args.layers and args.layers < cfg.n_layers:
        cfg = cfg.truncated(args.layers)
    if args.layers_dir:
        model = load_rank_model(cfg, args.layers_dir, world, rank, dev, cp=args.cp)      # streams the directory: one tensor on the host at a time
        epoch = f"ckpt:{os.path.abspath(args.layers_dir)}"
    else:
        model = random_rank_model(cfg, world, rank, dev, seed=args.seed)
        epoch = f"random:{args.seed}:{cfg.n_layers}"
    eng = DecodeEngine(rank, world, dev, cp=args.cp, ext=model, cfg=cfg, group=group, max_rows=8, cache_len=args.context + 1024)
    block = None
    if args.mode == "mtp":
        from ..mtp import MtpDraft
        from ..mtp.weights import load_mtp_files, random_mtp_checkpoint, shard_mtp

        if args.layers_dir and os.path.isfile(os.path.join(args.layers_dir, "mtp.safetensors")):
            draft = load_mtp_files(cfg, args.layers_dir, world, rank, dev, model["head"])
            epoch += "+mtp"
        else:                               # no draft weights: a random draft still yields the target's stream, at acceptance ~1
            draft = shard_mtp(random_mtp_checkpoint(cfg, seed=args.seed + 7, device=dev), cfg, world, rank, dev, model["head"])
            epoch += f"+mtp-random:{args.seed + 7}"
        block = MtpDraft(eng, draft)
    elif args.mode == "dflash":
        from dataclasses import replace

        from ..dflash import DFlashBlock, DFlashConfig
        from ..dflash.config import DFLASH_CONFIG, DFLASH_WEIGHTS
        from ..dflash.weights import load_dflash_files, load_dflash_shard, random_dflash_checkpoint

        real = DFLASH_CONFIG.is_file() and DFLASH_WEIGHTS.is_file()       # NEXRT_DFLASH_DIR / _CONFIG / _WEIGHTS
        dc = DFlashConfig.from_json(DFLASH_CONFIG) if real else DFlashConfig()
        if cfg.n_layers <= max(dc.target_layer_ids):      # truncated stack: tap the layers that exist
            step = max(cfg.n_layers // dc.n_taps, 1)
            dc = replace(dc, target_layer_ids=tuple(min(i * step, cfg.n_layers - 1) for i in range(dc.n_taps)))
        dc.validate_kernel_contract(cfg, world)
        if real:
            draft = load_dflash_files(dc, world, rank, dev, DFLASH_WEIGHTS)
            epoch += f"+dflash:{DFLASH_WEIGHTS}"
        else:
            draft = load_dflash_shard(random_dflash_checkpoint(dc, seed=args.seed + 11, device=dev), dc, world, rank, dev)
            epoch += f"+dflash-random:{args.seed + 11}"
        block = DFlashBlock(eng, dc, draft)
    return EngineBackend(eng, args.mode, block, model_epoch=epoch)


def queued_requests(args, vocab: int) -> List[Dict]:
    """Requests of the queue mode: ``--lens`` synthetic prompts (seeded uniform-random ids) and ``--files`` prompt
    texts, each with its own sampling seed ``seed_base + i``."""
    import glob
    import random

    out: List[Dict] = []
    for n in [int(v) for v in (args.lens or "").split(",") if v]:
        rnd = random.Random(n)
        out.append({"ids": [rnd.randrange(3, vocab) for _ in range(min(n, args.max_prompt))], "max_new": args.gen})
    for pattern in args.files or ():
        for path in sorted(glob.glob(pattern)):
            with open(path, encoding="utf-8") as f:
                out.append({"text": f.read(), "chat": True, "max_new": args.gen_files})
    for i, req in enumerate(out):
        req["seed"] = args.seed_base + i
    return out


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="nexrt_b200 bridge server (one process per GPU under torchrun)")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--listen", type=int, default=DEFAULT_PORT)
    p.add_argument("--mode", default="bs1", choices=["bs1", "mtp", "dflash"])
    p.add_argument("--layers", type=int, default=0)
    p.add_argument("--layers-dir", default=os.environ.get("NEXRT_LAYERS_DIR") if os.environ.get("NEXRT_LAYERS_DIR", "").startswith("/") and os.path.isdir(os.environ.get("NEXRT_LAYERS_DIR", "")) else None)
    p.add_argument("--tokenizer", default=os.environ.get("NEXRT_MODEL_DIR"))
    p.add_argument("--context", type=int, default=32768)
    p.add_argument("--cp", action="store_true")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--lens", default=None, help="comma list of synthetic prompt lengths served before listening")
    p.add_argument("--files", nargs="*", default=None, help="prompt files (globs) served before listening")
    p.add_argument("--gen", type=int, default=64, help="new tokens for --lens requests")
    p.add_argument("--gen-files", type=int, default=256, help="new tokens for --files requests")
    p.add_argument("--max-prompt", type=int, default=262080)
    p.add_argument("--seed-base", type=int, default=20260712, help="request i samples with seed base + i")
    p.add_argument("--verify", action="store_true", help="compare every stream with a plain one-row re-decode")
    p.add_argument("--cache-e2e", action="append", default=None, metavar="BASE,TARGET")
    p.add_argument("--cache-e2e-repetitions", type=int, default=3)
    p.add_argument("--cache-e2e-gen", type=int, default=8)
    p.add_argument("--cache-consensus-fault-rank", type=int, default=None, help="test only: this rank rejects its READY boundary once")
    p.add_argument("--no-listen", action="store_true", help="exit after the queued work")
    p.add_argument("--wide-prefill", type=int, default=int(os.environ.get("NEXRT_WIDE_PREFILL", "0") or 0),
                   help="rows per wide prefill chunk (16..128, a multiple of 8; every decode mode); 0 = 8-row steps")
    p.add_argument("--wide-terms", type=int, choices=(1, 2, 3), default=int(os.environ.get("NEXRT_WIDE_TERMS", "3") or 3),
                   help="e4m3 terms per activation of the wide prefill: 3 = the decode kernels' exact split, 1 = one plane (faster, FP8-rounded)")
    args = p.parse_args(argv)
    if args.wide_prefill and (args.wide_prefill % 8 or not 16 <= args.wide_prefill <= 128):
        p.error("--wide-prefill must be 0 or a multiple of 8 between 16 and 128")
    os.environ["NEXRT_WIDE_PREFILL"] = str(args.wide_prefill)      # read by DecodeEngine.prefill
    os.environ["NEXRT_WIDE_TERMS"] = str(args.wide_terms)          # read by DecodeEngine.wide_path
    import torch
    import torch.distributed as dist

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    ctl_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        ctl_group = dist.new_group(backend="gloo")
    backend = build_backend(args, rank, world, dev, None)
    server = BridgeServer(backend, load_tokenizer(args.tokenizer), rank, world, ctl_group, args.mode,
                          consensus_fault_rank=args.cache_consensus_fault_rank, verify=args.verify,
                          model_dir=args.tokenizer if args.tokenizer and os.path.isdir(args.tokenizer) else None)
    queue = queued_requests(args, backend.vocab)
    if queue:
        server.run_queue(queue)
    for pair in args.cache_e2e or ():
        base, target = (int(v) for v in pair.split(","))
        result = server.cache_e2e(base, target, args.cache_e2e_repetitions, args.cache_e2e_gen)
        if rank == 0:
            print("@@ CACHE-E2E " + json.dumps(result), flush=True)
    if not args.no_listen:
        server.serve_forever(args.host, args.listen)
    return 0


if __name__ == "__main__":
    sys.exit(main())
