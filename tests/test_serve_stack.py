"""Serving stack on CPU: failure policy, stream protocol, chunked prefill driver, the per-request
pipeline against a fake decode back end (single rank over a real socket, and several emulated ranks
sharing an in-process gather), request validation, client and launch-geometry checks."""

import json
import socket
import threading

import pytest

from nexrt_b200.serve import bridge_client
from nexrt_b200.serve.bridge import PrefillSession, chunked_prefill
from nexrt_b200.serve.bridge_serve import BadRequest, BridgeServer, ByteTokenizer, validate_request
from nexrt_b200.serve.cache_consensus import FatalTPInvariantError, RecoverableRequestError
from nexrt_b200.serve.cache_lifecycle import CacheBoundary, CachePhase
from nexrt_b200.serve.process_supervisor import launch_geometry, terminate_group
from nexrt_b200.serve.serve_control import (CacheReusePolicyError, FatalBackendError, RequestResetError, cache_key_for_request,
                                            dispatch_port_request, execute_request_with_consensus, is_fatal_backend_error)
from nexrt_b200.serve.stream_protocol import BridgeStreamWriter, IncrementalDetokenizer, decode_visible_text, visible_token_ids


# ---- a deterministic stand-in for the engine ----------------------------------------------------------
def _next(tokens):
    """Next token = hash of the whole history (so a wrong resume shows up as a different token)."""
    h = 17
    for t in tokens:
        h = (h * 31 + int(t)) % 250
    return h + 3


class FakeEngine:
    """Mimics the slice of DecodeEngine that the prefill driver uses."""

    def __init__(self):
        self.tokens, self.pending, self.evaluated = [], -1, 0

    def prefill(self, ids, chunk=8, resume_from=0, on_chunk=None):
        if resume_from:
            assert self.tokens == list(ids[:resume_from])
        else:
            self.tokens = []
        pos = resume_from
        while pos < len(ids):
            n = min(chunk, len(ids) - pos)
            self.tokens += list(ids[pos:pos + n])
            self.evaluated += n
            if on_chunk:
                on_chunk(pos, pos + n)
            pos += n
        self.pending = _next(self.tokens)
        return self.pending

    def _snapshot(self):
        return (list(self.tokens), self.pending)

    def _restore(self, snap):
        self.tokens, self.pending = list(snap[0]), snap[1]


class FakeBackend:
    vocab, capacity, model_epoch = 256 + 3, 128, "fake"

    def __init__(self, fail_decode=None, lose_boundary=False):
        self.eng, self.fail_decode, self.lose_boundary = FakeEngine(), fail_decode, lose_boundary
        self.sampling, self.resets, self._status = None, 0, 0

    def set_sampling(self, *a):
        self.sampling = a

    def prefill(self, tokens, resume, on_chunk):
        _, s = chunked_prefill(self.eng, tokens, 4, on_chunk=lambda s, e, nt: on_chunk(s, e) if e > s else None, resume=resume, return_session=True)
        return s

    def boundary(self):
        return CacheBoundary(len(self.eng.tokens), self.eng.pending, 0)

    def restore(self, session):
        self.eng._restore(session.snapshot)
        if self.lose_boundary:
            self.eng.pending ^= 1
        return self.boundary()

    def decode(self, max_new, eos_ids, on_tokens):
        if self.fail_decode is not None:
            raise self.fail_decode
        out = []
        for _ in range(max_new):
            t = self.eng.pending
            self.eng.tokens.append(t)
            self.eng.pending = _next(self.eng.tokens)
            out.append(self.eng.pending)
            on_tokens([self.eng.pending])
            if self.eng.pending in eos_ids:
                break
        return {"tokens": out, "rounds": len(out), "accept_mean": 1.0}

    def status(self):
        return self._status

    def reset(self, reason, cache, runtime_state):
        self.resets += 1
        cache.invalidate(reason, force=True)


def _req(**kw):
    base = {"text": "hello world", "max_new": 6, "cache_key": "k"}
    base.update(kw)
    return validate_request(base, 128, "bs1")


def _expected(prompt_ids, n):
    hist, out = list(prompt_ids), []
    for _ in range(n):
        t = _next(hist)
        out.append(t)
        hist.append(t)
    return out


# ---- serve_control ------------------------------------------------------------------------------------
def test_cache_key_policy_and_fatal_classification():
    assert cache_key_for_request("k", speculative=False) == "k"
    assert cache_key_for_request(None, speculative=True) is None
    with pytest.raises(CacheReusePolicyError):
        cache_key_for_request("k", speculative=True)
    assert is_fatal_backend_error(FatalBackendError("x"))
    assert is_fatal_backend_error(RuntimeError("CUDA error: an illegal memory access was encountered"))
    assert is_fatal_backend_error(RuntimeError("NCCL error in: something"))
    assert not is_fatal_backend_error(ValueError("collective mismatch in my own text"))
    assert not is_fatal_backend_error(KeyError("x"))


def test_execute_request_with_consensus_outcomes():
    life = lambda: (3, 2, 3, 0)  # noqa: E731
    resets = []
    ok = execute_request_with_consensus(lambda: {"v": 1}, lifecycle_state=life, gather_outcome=lambda r: [r, r], reset_request=resets.append)
    assert ok == {"v": 1} and not resets

    def recoverable():
        raise RecoverableRequestError("nope")

    with pytest.raises(RequestResetError):
        execute_request_with_consensus(recoverable, lifecycle_state=life, gather_outcome=lambda r: [r, r], reset_request=resets.append)
    assert resets == ["nope"]
    # this rank failed, the other succeeded -> fatal
    with pytest.raises(FatalTPInvariantError):
        execute_request_with_consensus(recoverable, lifecycle_state=life, gather_outcome=lambda r: [r, (2,) + tuple(r[1:])], reset_request=resets.append)
    with pytest.raises(FatalBackendError):
        execute_request_with_consensus(lambda: (_ for _ in ()).throw(RuntimeError("CUDA error: launch failed")), lifecycle_state=life,
                                       gather_outcome=lambda r: [r], reset_request=resets.append)
    with pytest.raises(FatalTPInvariantError):
        execute_request_with_consensus(lambda: (_ for _ in ()).throw(KeyError("bug")), lifecycle_state=life, gather_outcome=lambda r: [r],
                                       reset_request=resets.append)


class _Conn:
    def __init__(self):
        self.sent, self.closed = b"", False

    def sendall(self, b):
        self.sent += b

    def close(self):
        self.closed = True

    def settimeout(self, t):
        pass

    def shutdown(self, how):
        pass


def test_dispatch_port_request_paths():
    conn, report, fatal = _Conn(), [], []
    dispatch_port_request(lambda: {"tokens": [1]}, tp_rank=0, conn=conn, event_stream=None, report=report, terminate_fatally=lambda e, c: fatal.append(e))
    assert json.loads(conn.sent) == {"tokens": [1]} and conn.closed and report == [{"tokens": [1]}]
    conn = _Conn()
    dispatch_port_request(lambda: (_ for _ in ()).throw(RequestResetError("r")), tp_rank=0, conn=conn, event_stream=None, report=report,
                          terminate_fatally=lambda e, c: fatal.append(e))
    assert "error" in json.loads(conn.sent) and not fatal
    conn = _Conn()
    with pytest.raises(AssertionError):   # terminate_fatally must not return
        dispatch_port_request(lambda: (_ for _ in ()).throw(FatalBackendError("dead")), tp_rank=0, conn=conn, event_stream=None, report=report,
                              terminate_fatally=lambda e, c: fatal.append(e))
    assert isinstance(fatal[0], FatalBackendError) and conn.closed
    # other ranks never write
    dispatch_port_request(lambda: {"tokens": [2]}, tp_rank=1, conn=None, event_stream=None, report=report, terminate_fatally=lambda e, c: None)
    assert len(report) == 1


# ---- stream protocol ----------------------------------------------------------------------------------
def test_incremental_detokenizer_handles_split_utf8_and_stop_ids():
    tok = ByteTokenizer()
    ids = tok.encode("naïve ✓ done")
    det = IncrementalDetokenizer(tok, stop_ids=(2,))
    text = "".join(det.push([t]) for t in ids) + det.finish()
    assert text == "naïve ✓ done" and "�" not in text
    assert visible_token_ids(ids + [2, 5, 6], (2,)) == ids
    assert decode_visible_text(tok, ids + [2], (2,)) == "naïve ✓ done"


def test_stream_writer_emits_deltas_then_done():
    a, b = socket.socketpair()
    w = BridgeStreamWriter(a, ByteTokenizer(), stop_ids=(2,))
    ids = ByteTokenizer().encode("héllo")
    for t in ids:
        assert w.tokens([t])
    assert w.finish({"tokens": ids, "generated_text": "héllo", "status": 0})
    assert w.close()
    a.close()
    events = [json.loads(line) for line in b.makefile("rb").read().decode().splitlines()]
    assert "".join(e["text"] for e in events if e["type"] == "delta") == "héllo"
    assert events[-1]["type"] == "done" and "generated_text" not in events[-1]
    assert not w.tokens([5])          # closed writers refuse more output


def test_stream_writer_survives_a_client_that_stops_reading():
    a, b = socket.socketpair()
    w = BridgeStreamWriter(a, ByteTokenizer(), max_backlog=4, write_timeout=0.05, shutdown_timeout=0.1)
    b.close()
    for _ in range(64):
        w.tokens([70])
    w.finish({"tokens": []})
    w.close()
    assert w.stopped.wait(2.0)


# ---- chunked prefill driver ---------------------------------------------------------------------------
def test_chunked_prefill_resume_evaluates_only_the_suffix():
    eng, calls = FakeEngine(), []
    first, sess = chunked_prefill(eng, list(range(10)), 4, on_chunk=lambda s, e, nt: calls.append((s, e, nt)), return_session=True)
    assert calls == [(0, 4, -1), (4, 8, -1), (8, 10, first)] and first == _next(range(10)) and eng.evaluated == 10
    eng.tokens += [99]  # decode moved on; resume restores the boundary first
    first2, sess2 = chunked_prefill(eng, list(range(13)), 4, resume=sess, return_session=True)
    assert eng.evaluated == 13 and first2 == _next(range(13)) and sess2.tokens == tuple(range(13))
    # HIT: nothing to evaluate, same first token
    assert chunked_prefill(eng, list(range(13)), 4, resume=sess2) == first2 and eng.evaluated == 13
    with pytest.raises(ValueError):
        chunked_prefill(eng, [0, 1, 7], 4, resume=sess)
    with pytest.raises(TypeError):
        chunked_prefill(eng, [0, 1], 4, resume=object())
    with pytest.raises(ValueError):
        chunked_prefill(eng, [], 4)
    with pytest.raises(ValueError):
        chunked_prefill(eng, [1], 0)
    assert chunked_prefill(eng, [1, 2], 4, sample_next_token=lambda: 55) == 55


# ---- request validation ----------------------------------------------------------------------------------
@pytest.mark.parametrize("bad", [
    [], {"text": "a", "ids": [1]}, {}, {"text": 5}, {"ids": []}, {"ids": [1, -2]}, {"ids": [True]}, {"text": "a", "max_new": 0},
    {"text": "a", "max_new": True}, {"text": "a", "seed": -1}, {"text": "a", "seed": 1 << 64}, {"text": "a", "bogus": 1},
    {"text": "a", "temperature": -1}, {"text": "a", "top_p": 0}, {"text": "a", "top_k": 0}, {"text": "a", "cache_key": ""},
])
def test_validate_request_rejects(bad):
    with pytest.raises(BadRequest):
        validate_request(bad, 128, "bs1")


def test_validate_request_normalises_and_applies_mode_policy():
    r = validate_request({"text": "a"}, 128, "bs1")
    assert (r["max_new"], r["seed"], r["top_k"], r["stream"], r["cache_key"]) == (128, 0, 20, False, None)
    assert (r["temperature"], r["top_p"]) == pytest.approx((0.6, 0.95), rel=1e-6)
    assert validate_request({"cmd": "shutdown"}, 128, "bs1") == {"cmd": "shutdown"}
    assert validate_request({"text": "a", "seed": (1 << 64) - 1}, 128, "bs1")["seed"] == (1 << 64) - 1
    with pytest.raises(BadRequest):
        validate_request({"text": "a", "top_k": 5}, 128, "mtp")
    with pytest.raises(BadRequest):
        validate_request({"text": "a", "cache_key": "k"}, 128, "dflash")
    assert validate_request({"text": "a", "temperature": 0.0}, 128, "mtp")["temperature"] == 0.0


# ---- the request pipeline ----------------------------------------------------------------------------------
def test_pipeline_prefill_hit_append_and_token_stream():
    srv = BridgeServer(FakeBackend(), ByteTokenizer(), log=lambda *_: None)
    tok = srv.tok
    p1 = tok.encode("hello world")
    r1 = srv.run_request(_req(), p1)
    assert r1["cache"] == "prefill" and r1["tokens"] == _expected(p1, 6) and r1["stop_reason"] == "length" and r1["status"] == 0
    assert srv.state.cache.snapshot().phase == CachePhase.READY and srv.backend.eng.evaluated == len(p1)
    r2 = srv.run_request(_req(), p1)
    assert r2["cache"] == "hit" and r2["tokens"] == r1["tokens"] and srv.backend.eng.evaluated == len(p1)
    p3 = tok.encode("hello world, again")
    r3 = srv.run_request(_req(text="hello world, again"), p3)
    assert r3["cache"] == "append" and r3["tokens"] == _expected(p3, 6) and srv.backend.eng.evaluated == len(p3)
    # another owner, or no owner: full prefill; anonymous boundaries are not retained
    r4 = srv.run_request(_req(cache_key="other"), p1)
    assert r4["cache"] == "prefill"
    r5 = srv.run_request(_req(cache_key=None), p1)
    assert r5["cache"] == "prefill" and srv.state.cache.snapshot().phase == CachePhase.EMPTY
    assert srv.backend.sampling == pytest.approx((0, 0.6, 0.95, 20), rel=1e-6)


def test_pipeline_drops_a_boundary_that_was_not_restored():
    srv = BridgeServer(FakeBackend(lose_boundary=True), ByteTokenizer(), log=lambda *_: None)
    ids = srv.tok.encode("abc")
    r = srv.run_request(_req(text="abc"), ids)
    assert r["tokens"] == _expected(ids, 6)
    assert srv.state.cache.snapshot().phase == CachePhase.EMPTY and srv.state.session is None
    assert srv.run_request(_req(text="abc"), ids)["cache"] == "prefill"


def test_pipeline_recoverable_failure_resets_and_next_request_works():
    be = FakeBackend(fail_decode=RecoverableRequestError("sampler refused"))
    srv = BridgeServer(be, ByteTokenizer(), log=lambda *_: None)
    ids = srv.tok.encode("abc")
    with pytest.raises(RequestResetError):
        srv.run_request(_req(text="abc"), ids)
    assert be.resets == 1 and srv.state.cache.snapshot().phase == CachePhase.EMPTY and srv.state.session is None
    be.fail_decode = None
    assert srv.run_request(_req(text="abc"), ids)["tokens"] == _expected(ids, 6)
    be.fail_decode = RuntimeError("CUDA error: unspecified launch failure")
    with pytest.raises(FatalBackendError):
        srv.run_request(_req(text="abc"), ids)


def test_emulated_ranks_agree_or_fall_back_to_prefill_together():
    world = 3
    barrier, rows, lock = threading.Barrier(world), {}, threading.Lock()

    def make_gather(rank):
        def gather(rec):
            with lock:
                rows[rank] = tuple(rec)
            barrier.wait(10)
            table = [rows[r] for r in range(world)]
            barrier.wait(10)
            return table
        return gather

    servers = [BridgeServer(FakeBackend(), ByteTokenizer(), rank=r, world=world, gather=make_gather(r), log=lambda *_: None) for r in range(world)]
    ids = ByteTokenizer().encode("shared prompt")

    def run_all(req):
        out, errs = [None] * world, []

        def work(r):
            try:
                out[r] = servers[r].run_request(req, ids)
            except BaseException as e:  # noqa: BLE001
                errs.append(e)
                barrier.abort()

        ts = [threading.Thread(target=work, args=(r,)) for r in range(world)]
        [t.start() for t in ts]
        [t.join(20) for t in ts]
        assert not errs, errs
        return out

    first = run_all(_req(text="shared prompt"))
    assert {tuple(r["tokens"]) for r in first} == {tuple(_expected(ids, 6))} and {r["cache"] for r in first} == {"prefill"}
    # rank 1's device boundary drifts: every rank must take the PREFILL branch together
    servers[1].backend.eng.pending ^= 1
    second = run_all(_req(text="shared prompt"))
    assert {r["cache"] for r in second} == {"prefill"} and all(r["forced_prefill"] for r in second)
    third = run_all(_req(text="shared prompt"))
    assert {r["cache"] for r in third} == {"hit"}


def test_socket_server_end_to_end_with_client_and_stream():
    srv = BridgeServer(FakeBackend(), ByteTokenizer(), log=lambda *_: None)
    port_box, ready = [], threading.Event()
    t = threading.Thread(target=srv.serve_forever, kwargs=dict(port=0, ready=lambda p: (port_box.append(p), ready.set())), daemon=True)
    t.start()
    assert ready.wait(10)
    port = port_box[0]
    ids = ByteTokenizer().encode("ping")
    r = bridge_client.send_request({"text": "ping", "max_new": 5, "cache_key": "c"}, port=port, timeout=10)
    assert r["tokens"] == _expected(ids, 5) and r["prompt_tokens"] == 4
    bad = bridge_client.send_request({"text": "ping", "max_new": 0}, port=port, timeout=10)
    assert "bad request" in bad["error"]
    too_long = bridge_client.send_request({"ids": [5] * 200}, port=port, timeout=10)
    assert "exceeds" in too_long["error"]
    # nothing a client sends takes the server down: malformed fields, a prompt the chat template cannot take, raw garbage
    for junk in ({"messages": 5}, {"messages": [{"role": "user"}]}, {"messages": [None]}, {"text": "a", "chat": [1]}, {"ids": [1 << 70]}, [1, 2], "x", None):
        assert "bad request" in bridge_client.send_request(junk, port=port, timeout=10)["error"], junk
    with socket.create_connection(("127.0.0.1", port), timeout=10) as raw:
        raw.sendall(b"\xff\xfe not json at all\n")
        assert b"bad request" in raw.recv(1 << 16)
    events = list(bridge_client.stream_request({"text": "ping", "max_new": 5, "cache_key": "c"}, port=port, timeout=10))
    assert events[-1]["type"] == "done" and events[-1]["cache"] == "hit" and events[-1]["tokens"] == r["tokens"]
    assert "".join(e["text"] for e in events if e["type"] == "delta") == decode_visible_text(ByteTokenizer(), r["tokens"], (2,))
    assert bridge_client.send_request({"cmd": "shutdown"}, port=port, timeout=10) == {"ok": True}
    t.join(10)
    assert not t.is_alive()


# ---- launch geometry ------------------------------------------------------------------------------------
def test_launch_geometry_checks():
    assert launch_geometry(env={}) == (0, 1, 0)
    with pytest.raises(ValueError):
        launch_geometry(8, env={})
    env = {"RANK": "3", "WORLD_SIZE": "8", "LOCAL_RANK": "3", "LOCAL_WORLD_SIZE": "8"}
    assert launch_geometry(8, env=env) == (3, 8, 3)
    for patch in ({"WORLD_SIZE": "3", "LOCAL_WORLD_SIZE": "3"}, {"LOCAL_WORLD_SIZE": "4"}, {"RANK": "11"}, {"RANK": "x"}):
        with pytest.raises(ValueError):
            launch_geometry(None, env={**env, **patch})
    with pytest.raises(ValueError):
        launch_geometry(4, env=env)
    codes = []
    terminate_group("test", log=lambda m: None, exit_fn=codes.append)
    assert codes == [2]


# ---- two real processes over gloo ---------------------------------------------------------------------
def test_two_rank_server_over_gloo(tmp_path):
    """Rank 0 accepts, both ranks run the pipeline; rank 1 fails to restore its boundary after the first
    request, so the boundary is dropped by both and the repeat is a collective PREFILL, then a HIT."""
    import os
    import subprocess
    import sys
    import time

    port_file = str(tmp_path / "port")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "serve_worker.py")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE="2", LOCAL_WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, worker, port_file, "1"], env=dict(env, RANK=str(r), LOCAL_RANK=str(r))) for r in range(2)]
    try:
        deadline = time.time() + 120
        while not os.path.exists(port_file):
            assert time.time() < deadline and all(p.poll() is None for p in procs), "server did not come up"
            time.sleep(0.1)
        port = int(open(port_file).read())
        ids = ByteTokenizer().encode("two ranks")
        req = {"text": "two ranks", "max_new": 5, "cache_key": "c"}
        r1 = bridge_client.send_request(req, port=port, timeout=60)
        assert r1["tokens"] == _expected(ids, 5) and r1["cache"] == "prefill"
        r2 = bridge_client.send_request(req, port=port, timeout=60)
        assert r2["cache"] == "prefill" and r2["tokens"] == r1["tokens"]      # boundary was dropped by consensus
        r3 = bridge_client.send_request(req, port=port, timeout=60)
        assert r3["cache"] == "hit" and r3["tokens"] == r1["tokens"]
        assert bridge_client.send_request({"cmd": "shutdown"}, port=port, timeout=60) == {"ok": True}
        for p in procs:
            assert p.wait(60) == 0
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# ---- queue mode, cache matrix, injected consensus fault -------------------------------------------------------
def test_queue_mode_and_cache_matrix():
    import argparse

    from nexrt_b200.serve.bridge_serve import queued_requests

    args = argparse.Namespace(lens="5,9", files=None, gen=4, gen_files=8, max_prompt=7, seed_base=100)
    queue = queued_requests(args, FakeBackend.vocab)
    assert [len(r["ids"]) for r in queue] == [5, 7] and [r["seed"] for r in queue] == [100, 101] and queue == queued_requests(args, FakeBackend.vocab)
    srv = BridgeServer(FakeBackend(), ByteTokenizer(), log=lambda *_: None)
    out = srv.run_queue(queue)
    assert [r["request"] for r in out] == [0, 1] and all(len(r["tokens"]) == 4 and r["cache"] == "prefill" for r in out)
    res = srv.cache_e2e(6, 11, repetitions=2, gen=3)
    assert res["ok"] and [r["cache"] for r in res["rows"][:5]] == ["prefill", "hit", "append", "prefill", "prefill"]
    with pytest.raises(ValueError):
        srv.cache_e2e(5, 5)


def test_injected_boundary_fault_forces_one_collective_prefill():
    srv = BridgeServer(FakeBackend(), ByteTokenizer(), log=lambda *_: None, consensus_fault_rank=0)
    ids = srv.tok.encode("abc")
    assert srv.run_request(_req(text="abc"), ids)["cache"] == "prefill"
    r = srv.run_request(_req(text="abc"), ids)                       # would be a HIT; the injected fault rejects it
    assert r["cache"] == "prefill" and r["forced_prefill"]
    assert srv.run_request(_req(text="abc"), ids)["cache"] == "hit"   # injected once


def test_verify_gate_reports_a_mismatch():
    class Checking(FakeBackend):
        def verify_tokens(self, session, tokens, req):
            return list(tokens) == _expected(session.tokens, len(tokens)) and self.good

    be = Checking()
    be.good = True
    srv = BridgeServer(be, ByteTokenizer(), log=lambda *_: None, verify=True)
    ids = srv.tok.encode("abc")
    assert srv.run_request(_req(text="abc"), ids)["verified"] is True
    be.good = False
    assert srv.run_request(_req(text="abc"), ids)["verified"] is False
    assert BridgeServer(FakeBackend(), ByteTokenizer(), log=lambda *_: None).run_request(_req(text="abc"), ids)["verified"] is None


def test_worker_rejects_a_bad_wide_prefill_size(capsys):
    """The chunk size of the wide prefill path is checked before any engine is built."""
    from nexrt_b200.serve import bridge_serve

    for bad in ("12", "8", "136", "20"):
        with pytest.raises(SystemExit):
            bridge_serve.main(["--wide-prefill", bad, "--no-listen"])
    assert "--wide-prefill must be 0 or a multiple of 8" in capsys.readouterr().err


# ---- client command line (reference tests/test_bridge_client.py) ---------------------------------------------------
def _run_client(argv, reply=b'{"ok": true}\n'):
    """``bridge_client.main(argv)`` against a mocked socket: returns (exit code, request sent or None, connect calls)."""
    import contextlib
    import io
    from unittest.mock import MagicMock, patch

    conn = MagicMock()
    conn.__enter__.return_value = conn
    conn.recv.return_value = reply
    code, sent = None, None
    with patch.object(bridge_client.socket, "create_connection", return_value=conn) as connect, \
            contextlib.redirect_stdout(io.StringIO()), contextlib.redirect_stderr(io.StringIO()):
        try:
            code = bridge_client.main(["--port", "9411", *argv])
        except SystemExit as e:
            code = e.code
    if conn.sendall.call_args is not None:
        sent = json.loads(conn.sendall.call_args.args[0])
    return code, sent, connect.call_count


def test_client_reads_prompt_files_locally_and_sends_inline_text(tmp_path):
    path = tmp_path / "prompt.txt"
    text = "你好，NexRT\nSecond line."
    path.write_text(text, encoding="utf-8")
    code, sent, _ = _run_client(["--file", str(path), "--chat", "--max-new", "16", "--seed", "7"])
    assert code == 0 and sent == {"text": text, "chat": True, "max_new": 16, "seed": 7}
    code, sent, _ = _run_client(["--text", "hello", "--temperature", "0", "--top-p", "0.95", "--top-k", "28"])
    assert code == 0 and sent == {"text": "hello", "max_new": 128, "seed": 0, "temperature": 0.0, "top_p": 0.95, "top_k": 28}
    code, sent, _ = _run_client(["--ids", "5,6,7", "--cache-key", "k"])
    assert code == 0 and sent == {"ids": [5, 6, 7], "max_new": 128, "seed": 0, "cache_key": "k"}
    assert _run_client(["--shutdown"])[:2] == (0, {"cmd": "shutdown"})


def test_client_fails_before_connecting_when_the_file_cannot_be_read(tmp_path):
    code, sent, connects = _run_client(["--file", str(tmp_path / "missing.txt")])
    assert code == 2 and sent is None and connects == 0
    bad = tmp_path / "latin1.txt"
    bad.write_bytes(b"caf\xe9")
    assert _run_client(["--file", str(bad)])[0::2] == (2, 0)
    assert _run_client(["--file", str(bad), "--text", "x"])[0::2] == (2, 0)


def test_incremental_detokenizer_equals_one_shot_decode_on_any_byte_stream():
    """Streamed text == one-shot text for valid UTF-8 and for arbitrary bytes (a model can emit any byte-fallback token),
    in any grouping, with a bounded window; a run of invalid bytes longer than the window never raises (reference
    tests/test_openai_serve.py: test_incremental_detokenizer_matches_one_shot_with_bounded_state)."""
    import random

    tok = ByteTokenizer()
    rng = random.Random(0)
    for trial in range(600):
        n = rng.randint(0, 120)
        mode = rng.random()
        if mode < 0.4:
            ids = tok.encode("".join(rng.choice("aé✓😀\n z中") for _ in range(n)))
        elif mode < 0.7:
            ids = [3 + rng.randrange(256) for _ in range(n)]
        else:
            ids = [3 + rng.choice([0x80, 0xBF, 0xE2, 0xF0, 0x41]) for _ in range(n)]
        tail = rng.choice([4, 5, 8, 32])
        det = IncrementalDetokenizer(tok, max_tail_tokens=tail)
        out, i = "", 0
        while i < len(ids):
            g = rng.randint(1, 5)
            out += det.push(ids[i : i + g])
            i += g
            assert det.retained_tokens <= tail
        out += det.finish()
        assert out == decode_visible_text(tok, ids, ()), (trial, tail, ids[:24])
    # a character spread over more tokens than the window keeps: the window is flushed as it decodes, nothing raises
    det = IncrementalDetokenizer(tok, max_tail_tokens=1)
    text = "".join(det.push([t]) for t in tok.encode("a😀b")) + det.finish()
    assert text.startswith("a") and text.endswith("b")


def test_request_validation_survives_arbitrary_json():
    """Random request objects through ``validate_request`` and ``BridgeServer.tokenize``: the outcome is a normalised
    request with in-vocabulary ids, or ``BadRequest`` - never another exception (the accept loop would have to guess)."""
    import random

    rng = random.Random(1)
    srv = BridgeServer(FakeBackend(), ByteTokenizer(), log=lambda *_: None)

    def value(depth=0):
        c = rng.randrange(12)
        if c == 0:
            return None
        if c == 1:
            return rng.choice([True, False])
        if c == 2:
            return rng.choice([0, 1, -1, 5, 1 << 70, 255, 258, 259])
        if c == 3:
            return rng.choice([0.0, 1.5, float("nan"), float("inf"), -2.0, 1e40])
        if c == 4:
            return rng.choice(["", "a", "héllo", "x" * 200])
        if c == 5 and depth < 2:
            return [value(depth + 1) for _ in range(rng.randrange(4))]
        if c == 6 and depth < 2:
            return {rng.choice(["role", "content", "x"]): value(depth + 1) for _ in range(rng.randrange(3))}
        if c == 7:
            return [{"role": "user", "content": "hi"}]
        if c == 8:
            return [5, 6, 7]
        return rng.choice(["a", 3, 0.5])

    keys = ["text", "ids", "chat", "messages", "max_new", "seed", "cache_key", "temperature", "top_p", "top_k", "stream", "cmd", "bogus"]
    accepted = 0
    for _ in range(4000):
        roll = rng.random()
        if roll < 0.1:
            req = value()
        elif roll < 0.5:      # a valid request with one field replaced by something arbitrary
            req = dict(rng.choice([{"text": "héllo"}, {"ids": [5, 6, 7]}, {"messages": [{"role": "user", "content": "hi"}]}, {"text": "q", "chat": True}]),
                       max_new=4, seed=3)
            if rng.random() < 0.7:
                req[rng.choice(keys)] = value()
        else:
            req = {k: value() for k in rng.sample(keys, rng.randrange(0, 6))}
        for mode in ("bs1", "mtp"):
            try:
                r = validate_request(req, srv.backend.capacity, mode, srv.sampling)
                if r.get("cmd") == "shutdown":
                    continue
                ids = srv.tokenize(r)
            except BadRequest:
                continue
            accepted += 1
            assert ids and all(isinstance(t, int) and 0 <= t < srv.backend.vocab for t in ids)
            json.dumps(r)
    assert accepted > 20          # the generator does produce valid requests too


class _PausedConnection:
    """A connection whose first send blocks until released (a client that is slow, not gone)."""

    def __init__(self):
        self.started, self.release, self.writes = threading.Event(), threading.Event(), []

    def settimeout(self, t):
        pass

    def sendall(self, data):
        self.started.set()
        assert self.release.wait(10.0)
        self.writes.append(data)

    def shutdown(self, how):
        self.release.set()


def test_stream_writer_merges_tokens_behind_a_slow_send_and_keeps_the_terminal_event():
    """While one send is stuck, token events merge into one queued delta (no backlog slots), the terminal event still
    fits (reference tests/test_openai_serve.py: test_stream_writer_terminal_event_uses_one_backlog_slot), and the client
    gets the whole text once it reads again."""
    conn = _PausedConnection()
    tok = ByteTokenizer()
    w = BridgeStreamWriter(conn, tok, stop_ids=(2,), max_backlog=2, shutdown_timeout=2.0)
    assert w.event({"type": "start"})
    assert conn.started.wait(2.0)
    ids = tok.encode("slow but alive: " + "é✓" * 200)
    assert all(w.tokens([t]) for t in ids)                    # hundreds of callbacks, none refused, none blocking
    assert w.finish({"tokens": ids, "generated_text": "x", "status": 0})
    assert not w.tokens([5])
    conn.release.set()
    assert w.close() and not w.disconnected
    events = [json.loads(line) for data in conn.writes for line in data.decode().splitlines()]
    assert [e["type"] for e in events] == ["start", "delta", "done"]
    assert events[1]["text"] == decode_visible_text(tok, ids, (2,))
    # different kinds do not merge: two raw events behind a stuck send fill a backlog of two, the third offer drops the stream
    conn2 = _PausedConnection()
    w2 = BridgeStreamWriter(conn2, tok, max_backlog=2, shutdown_timeout=0.2)
    assert w2.event({"type": "start"}) and conn2.started.wait(2.0)
    assert w2.event({"a": 1}) and w2.event({"a": 2}) and not w2.event({"a": 3}) and w2.disconnected
    conn2.release.set()
    w2.close()
