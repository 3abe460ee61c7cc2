"""Host loop of a speculative request (``runtime/rounds.py``) against a scripted host mirror, and the server's stop-token
resolution (reference behaviour: tests/test_bridge_request_validation.py, test_model_and_tokenizer_eos_are_both_stops;
sglang_prefill/bridge_serve.py:140-165).  No GPU: the loop only replays a graph object and reads mirror words."""

import json
from types import SimpleNamespace

import pytest

from nexrt_b200.runtime.control import CTL_WORDS, Ctl
from nexrt_b200.runtime.rounds import consume_rounds, stop_set
from nexrt_b200.serve.bridge_serve import resolve_stop_ids


class ScriptedMirror:
    """Rounds are (tokens committed, status); generation numbers count launches, words are produced on wait."""

    def __init__(self, script, start_len=100):
        self.script, self.launched, self.waited, self.len = list(script), 0, [], start_len
        self.resyncs = 0

    def resync(self):
        self.resyncs += 1

    def next_gen(self):
        self.launched += 1
        return self.launched

    def wait(self, gen):
        self.waited.append(gen)
        toks, status = self.script[gen - 1] if gen - 1 < len(self.script) else ([7], 0)
        words = [0] * CTL_WORDS
        words[Ctl.STATUS], words[Ctl.COMMIT_COUNT] = status, len(toks)
        for i, t in enumerate(toks):
            words[Ctl.EMITTED + i] = t
        self.len += len(toks)
        words[Ctl.COMMITTED_LEN] = self.len
        return words


def fake_engine(script, budget=10_000, start_len=100):
    mirror = ScriptedMirror(script, start_len)
    graph = SimpleNamespace(replays=0)
    graph.replay = lambda: setattr(graph, "replays", graph.replays + 1)
    eng = SimpleNamespace(mirror=mirror, _kv_budget=lambda: budget)
    return eng, graph


def test_stop_set_forms():
    assert stop_set(None) == frozenset() and stop_set(5) == {5} and stop_set(-1) == frozenset()
    assert stop_set([3, None, 9, 3, -2]) == {3, 9} and stop_set(()) == frozenset()
    with pytest.raises(TypeError):
        stop_set(True)


def test_rounds_until_max_new_with_one_round_in_flight():
    eng, graph = fake_engine([([1, 2, 3], 0), ([4], 0), ([5, 6, 7, 8], 0), ([9], 0)])
    seen, stats = [], {}
    out = consume_rounds(eng, graph, max_new=6, on_tokens=seen.append, stats=stats, reserve=8)
    assert out == [1, 2, 3, 4, 5, 6]
    assert seen == [[1, 2, 3], [4], [5, 6]]                      # the callback sees what the request keeps, nothing past it
    assert stats["rounds"] == 3 and stats["accept_mean"] == pytest.approx(8 / 3)
    assert eng.mirror.resyncs == 1
    # every launched round was waited for before returning (at most one beyond the round that ended the request)
    assert sorted(eng.mirror.waited) == list(range(1, graph.replays + 1)) and graph.replays <= 4


@pytest.mark.parametrize("eos", [6, (99, 6), {6, 2000}])
def test_any_stop_id_ends_the_request_inside_a_round(eos):
    eng, graph = fake_engine([([1, 2], 0), ([5, 6, 7, 8], 0), ([9], 0)])
    seen = []
    out = consume_rounds(eng, graph, max_new=50, eos=eos, on_tokens=seen.append)
    assert out == [1, 2, 5, 6] and seen == [[1, 2], [5, 6]]
    assert sorted(eng.mirror.waited) == list(range(1, graph.replays + 1))


def test_failed_round_raises_after_draining_what_is_in_flight():
    eng, graph = fake_engine([([1], 0), ([], 3), ([2], 0)])
    with pytest.raises(RuntimeError, match="MTP round failed: status 3"):
        consume_rounds(eng, graph, max_new=10, what="MTP round")
    assert sorted(eng.mirror.waited) == list(range(1, graph.replays + 1))
    eng, graph = fake_engine([([], 0)])                       # a round that committed nothing is a failure too
    with pytest.raises(RuntimeError):
        consume_rounds(eng, graph, max_new=4)


def test_cache_end_stops_the_request():
    eng, graph = fake_engine([([1, 2, 3, 4], 0)] * 10, budget=120, start_len=100)
    out = consume_rounds(eng, graph, max_new=100, reserve=8)          # stops once the committed length reaches 112
    assert out == [1, 2, 3, 4] * 3
    assert consume_rounds(*fake_engine([([1], 0)]), max_new=0) == []


def test_generate_wrappers_pass_every_stop_id_through(monkeypatch):
    from nexrt_b200.dflash import serve as dserve
    from nexrt_b200.mtp import serve as mserve

    eng, graph = fake_engine([([1, 2], 0), ([3, 4], 0), ([5], 0)])
    assert mserve.generate_mtp(SimpleNamespace(eng=eng), graph, max_new=9, eos=[4, 77]) == [1, 2, 3, 4]
    eng, graph = fake_engine([([1, 2], 0), ([3, 4], 0), ([5], 0)])
    assert dserve.generate_dflash(SimpleNamespace(eng=eng), graph, max_new=9, eos=3) == [1, 2, 3]


def test_stop_ids_come_from_tokenizer_generation_config_and_tool_call_openers(tmp_path):
    tok = SimpleNamespace(eos_token_id=248046, unk_token_id=0, convert_tokens_to_ids=lambda text: 248058 if text == "<tool_call>" else 0)
    assert resolve_stop_ids(tok, str(tmp_path)) == (248046, 248058)          # no generation_config.json
    cfg = tmp_path / "generation_config.json"
    for eos in (248044, [248046, 248044, 248044]):
        cfg.write_text(json.dumps({"eos_token_id": eos}))
        assert resolve_stop_ids(tok, str(tmp_path)) == (248044, 248046, 248058)
    tok.eos_token_id = [248046, 248044]
    for eos in (None, []):
        cfg.write_text(json.dumps({"eos_token_id": eos}))
        assert resolve_stop_ids(tok, str(tmp_path)) == (248044, 248046, 248058)
    tok.eos_token_id = None
    assert resolve_stop_ids(tok, str(tmp_path)) == (248058,)
    cfg.write_text("{ not json")
    assert resolve_stop_ids(tok, str(tmp_path)) == (248058,)
    # a tokenizer without the conversion hook, or one that raises for unknown strings
    assert resolve_stop_ids(SimpleNamespace(eos_token_id=2)) == (2,)

    def boom(text):
        raise KeyError(text)

    assert resolve_stop_ids(SimpleNamespace(eos_token_id=[2, 5], unk_token_id=None, convert_tokens_to_ids=boom)) == (2, 5)


def test_stream_deltas_of_a_speculative_request_equal_the_final_text():
    """Rounds -> ``on_tokens`` -> stream writer: with a stop token in the middle of a round the concatenated deltas are
    exactly the visible text of the tokens the request returns (reference tests/test_stream_callbacks.py:
    test_mtp_stop_token_stream_deltas_equal_json_text)."""
    import socket

    from nexrt_b200.serve.bridge_serve import ByteTokenizer
    from nexrt_b200.serve.stream_protocol import BridgeStreamWriter, decode_visible_text

    tok = ByteTokenizer()
    ids = tok.encode("héllo wörld")
    stop = tok.eos_token_id
    script = [(ids[:3], 0), (ids[3:7], 0), (ids[7:] + [stop, ids[0], ids[1]], 0), ([ids[2]], 0)]
    eng, graph = fake_engine(script)
    a, b = socket.socketpair()
    try:
        w = BridgeStreamWriter(a, tok, stop_ids=(stop, 99999))
        out = consume_rounds(eng, graph, max_new=64, eos=(99999, stop), on_tokens=w.tokens)
        assert out == ids + [stop]
        text = decode_visible_text(tok, out, (stop, 99999))
        assert w.finish({"tokens": out, "generated_text": text, "status": 0}) and w.close()
        a.close()
        events = [json.loads(line) for line in b.makefile("rb").read().decode().splitlines()]
    finally:
        b.close()
    assert text == "héllo wörld" and "".join(e["text"] for e in events if e["type"] == "delta") == text
    assert events[-1]["type"] == "done"
