"""Sampling ABI and the CPU oracle (reference tests/test_sampling.py, test_seed_width.py)."""

import struct

import pytest

from nexrt_b200.sampling import (checked_sampling_config, resolve_sampling_config, sample_reference, sampling_words,
                                 seeded_uniform, splitmix64)


def test_words_layout():
    w = sampling_words(42, 0.6, 0.95, 20)
    assert len(w) == 8 and w[0] == 42 and w[2] == 20 and w[3:] == [0] * 5
    t, p = struct.unpack("<ff", struct.pack("<q", w[1]))
    assert abs(t - 0.6) < 1e-6 and abs(p - 0.95) < 1e-6


def test_seed_is_full_64_bit():
    big = (1 << 64) - 5
    w = sampling_words(big, 0.0, 1.0, 1)
    assert w[0] == -5 and (w[0] & ((1 << 64) - 1)) == big


@pytest.mark.parametrize("bad", [(-1, 0.9, 5), (float("nan"), 0.9, 5), (0.5, 0.0, 5), (0.5, 1.5, 5), (0.5, 0.9, 0), (0.5, 0.9, 29),
                                 (0.5, 0.9, True), (0.5, 0.9, 2.5), (1e-50, 0.9, 5)])
def test_rejects_bad_config(bad):
    with pytest.raises(ValueError):
        checked_sampling_config(*bad)


def test_resolve_defaults():
    assert resolve_sampling_config((0.6, 0.95, 20), top_k=3)[2] == 3


def test_splitmix_known_values():
    assert splitmix64(0) == 0xE220A8397B1DCDAF
    u = seeded_uniform(42, 7)
    assert 0.0 <= u < 1.0 and u == seeded_uniform(42, 7) and u != seeded_uniform(42, 8)


def test_reference_sampler_greedy_and_ties():
    logits = [0.0, 3.0, 3.0, 1.0]
    tok, kept, probs = sample_reference(logits, 1, 0, 0.0, 1.0, 1)
    assert tok == 1 and kept == [1]
    tok, kept, probs = sample_reference(logits, 1, 0, 1.0, 1.0, 3)
    assert kept[:2] == [1, 2] and abs(sum(probs) - 1.0) < 1e-9 and tok in kept


def test_model_generation_config_sets_the_server_defaults(tmp_path, monkeypatch):
    """``generation_config.json`` of the model directory over the built-in defaults, request values over both;
    ``do_sample: false`` means greedy whatever else the file says (reference tests/test_sampling.py:
    test_model_defaults_and_request_overrides)."""
    import json

    from nexrt_b200.sampling import DEFAULT_SAMPLING, resolve_sampling_config, sampling_defaults

    for var in ("NEXRT_MODEL_DIR", "NEXRT_LAYERS_DIR"):
        monkeypatch.delenv(var, raising=False)
    assert sampling_defaults() == pytest.approx(DEFAULT_SAMPLING) and sampling_defaults(str(tmp_path)) == pytest.approx(DEFAULT_SAMPLING)    # float32-rounded
    path = tmp_path / "generation_config.json"
    path.write_text(json.dumps(dict(temperature=0.7, top_p=0.9, top_k=28)))
    defaults = sampling_defaults(str(tmp_path))
    assert defaults == pytest.approx((0.7, 0.9, 28))
    monkeypatch.setenv("NEXRT_MODEL_DIR", str(tmp_path))
    assert sampling_defaults() == defaults
    assert resolve_sampling_config(defaults, temperature=0) == (0, defaults[1], 28) and resolve_sampling_config(defaults) == defaults
    path.write_text(json.dumps(dict(do_sample=False, temperature=1, top_k=50)))
    assert sampling_defaults()[::2] == (0, 1)


def test_server_applies_the_model_defaults_to_requests(tmp_path):
    import json

    from nexrt_b200.serve.bridge_serve import BridgeServer, ByteTokenizer, validate_request

    (tmp_path / "generation_config.json").write_text(json.dumps(dict(temperature=0.3, top_p=0.8, top_k=7, eos_token_id=[2, 9])))
    backend = type("B", (), {"capacity": 64, "model_epoch": "m", "vocab": 300})()
    srv = BridgeServer(backend, ByteTokenizer(), log=lambda *_: None, model_dir=str(tmp_path))
    assert srv.sampling == pytest.approx((0.3, 0.8, 7)) and srv.stop_ids == (2, 9)
    req = validate_request({"text": "a"}, 64, "bs1", srv.sampling)
    assert (req["temperature"], req["top_p"], req["top_k"]) == pytest.approx((0.3, 0.8, 7))
    req = validate_request({"text": "a", "temperature": 0.0, "top_k": 3}, 64, "bs1", srv.sampling)
    assert (req["temperature"], req["top_p"], req["top_k"]) == pytest.approx((0.0, 0.8, 3))
