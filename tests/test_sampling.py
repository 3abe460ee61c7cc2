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
