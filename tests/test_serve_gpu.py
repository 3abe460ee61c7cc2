"""The request pipeline over the real engine (shrunk model, one GPU): a retained prompt boundary must
give the same tokens as a fresh prefill (HIT and APPEND), decode must leave the boundary restorable,
and streaming must deliver the same text as the final reply.  Mirrors the reference's cache
end-to-end test (nex_n2_5_pro/tests/test_bridge_cache_e2e.py) without SGLang."""

import json
import socket

import pytest

from nexrt_b200.models.reference import synthetic_prompt
from nexrt_b200.serve.bridge_serve import BridgeServer, ByteTokenizer, EngineBackend, validate_request
from nexrt_b200.serve.cache_lifecycle import CachePhase
from nexrt_b200.serve.stream_protocol import BridgeStreamWriter
from nexrt_b200.testing import make_engine, shrunk_checkpoint

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def server():
    cfg, ckpt = shrunk_checkpoint(0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    return BridgeServer(EngineBackend(eng, "bs1", chunk=8, model_epoch="shrunk:0"), ByteTokenizer(), log=lambda *_: None)


def _req(ids, **kw):
    base = {"ids": ids, "max_new": 8, "temperature": 0.0, "cache_key": "k"}
    base.update(kw)
    return validate_request(base, 4096, "bs1")


def test_hit_and_append_reproduce_a_fresh_prefill(server):
    cfg = server.backend.eng.cfg
    base = synthetic_prompt(cfg.vocab, 40, seed=3)
    longer = base + synthetic_prompt(cfg.vocab, 13, seed=4)
    fresh_base = server.run_request(_req(base, cache_key=None), base)
    fresh_long = server.run_request(_req(longer, cache_key=None), longer)
    assert fresh_base["cache"] == fresh_long["cache"] == "prefill" and fresh_base["status"] == 0
    assert len(fresh_base["tokens"]) == 8 and server.state.cache.snapshot().phase == CachePhase.EMPTY
    r1 = server.run_request(_req(base), base)
    assert r1["cache"] == "prefill" and r1["tokens"] == fresh_base["tokens"]
    assert server.state.cache.snapshot().phase == CachePhase.READY
    r2 = server.run_request(_req(base), base)
    assert r2["cache"] == "hit" and r2["tokens"] == fresh_base["tokens"]
    r3 = server.run_request(_req(longer), longer)
    assert r3["cache"] == "append" and r3["tokens"] == fresh_long["tokens"]
    # a shorter prompt can never reuse the boundary (the recurrent state cannot be rewound)
    r4 = server.run_request(_req(base), base)
    assert r4["cache"] == "prefill" and r4["tokens"] == fresh_base["tokens"]


def test_sampled_requests_are_reproducible_per_seed(server):
    cfg = server.backend.eng.cfg
    ids = synthetic_prompt(cfg.vocab, 24, seed=5)
    a = server.run_request(_req(ids, temperature=1.0, top_p=0.95, top_k=20, seed=11, cache_key=None), ids)
    b = server.run_request(_req(ids, temperature=1.0, top_p=0.95, top_k=20, seed=11, cache_key=None), ids)
    c = server.run_request(_req(ids, temperature=1.0, top_p=0.95, top_k=20, seed=12, cache_key=None), ids)
    assert a["tokens"] == b["tokens"] and a["status"] == 0
    assert a["tokens"] != c["tokens"]


def test_streamed_text_equals_the_final_text(server):
    ids = [t + 3 for t in b"stream me"]
    a, b = socket.socketpair()
    w = BridgeStreamWriter(a, server.tok, server.stop_ids)
    res = server.run_request(_req(ids, cache_key=None), ids, stream=w)
    w.finish(res)
    assert w.close()
    a.close()
    events = [json.loads(x) for x in b.makefile("rb").read().decode().splitlines()]
    assert events[-1]["type"] == "done" and events[-1]["tokens"] == res["tokens"]
    assert "".join(e["text"] for e in events if e["type"] == "delta") == res["generated_text"]


def test_verify_gate_and_cache_matrix_on_the_engine(server):
    cfg = server.backend.eng.cfg
    server.verify = True
    try:
        ids = synthetic_prompt(cfg.vocab, 20, seed=8)
        r = server.run_request(_req(ids, cache_key=None), ids)
        assert r["verified"] is True and r["status"] == 0
    finally:
        server.verify = False
    res = server.cache_e2e(24, 37, repetitions=1, gen=6)
    assert res["ok"], res


def test_wide_prefill_boundary_is_reusable(server, monkeypatch):
    """Prompts prefilled in wide chunks leave a boundary that HIT and APPEND requests continue from."""
    monkeypatch.setenv("NEXRT_WIDE_PREFILL", "16")
    cfg = server.backend.eng.cfg
    base = synthetic_prompt(cfg.vocab, 45, seed=21)
    longer = base + synthetic_prompt(cfg.vocab, 20, seed=22)
    r1 = server.run_request(_req(base, cache_key="w"), base)
    assert r1["cache"] == "prefill" and r1["status"] == 0 and len(r1["tokens"]) == 8
    assert any(key[0] == 16 for key in server.backend.eng._wide)                       # the wide path ran
    r2 = server.run_request(_req(base, cache_key="w"), base)
    assert r2["cache"] == "hit" and r2["tokens"] == r1["tokens"]
    r3 = server.run_request(_req(longer, cache_key="w"), longer)
    assert r3["cache"] == "append" and r3["status"] == 0 and len(r3["tokens"]) == 8
