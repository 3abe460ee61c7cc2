"""Determinism: the same request twice gives bitwise-identical logits and tokens (eager and graph
replay), independent of what ran in between - every reduction in the step has a fixed order."""

import pytest
import torch

from nexrt_b200.models.reference import synthetic_prompt
from nexrt_b200.testing import gather_logits, make_engine, shrunk_checkpoint

pytestmark = pytest.mark.gpu


def _run(eng, prompt, n_new):
    first = eng.prefill(prompt, chunk=8)
    rows = gather_logits(eng, 8).clone()
    toks = [first] + eng.generate(max_new=n_new)
    return rows, toks


def test_repeat_runs_are_bitwise_identical():
    cfg, ckpt = shrunk_checkpoint(0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    eng.head.enable_logits()
    prompt = synthetic_prompt(cfg.vocab, 40, seed=21)
    other = synthetic_prompt(cfg.vocab, 23, seed=22)
    a_rows, a_toks = _run(eng, prompt, 12)
    _run(eng, other, 5)                                   # unrelated request in between
    b_rows, b_toks = _run(eng, prompt, 12)
    assert a_toks == b_toks and torch.equal(a_rows, b_rows)
    # a second engine instance (fresh buffers, fresh graphs) agrees bit for bit as well
    eng2 = make_engine(cfg, ckpt, max_rows=8)
    eng2.head.enable_logits()
    c_rows, c_toks = _run(eng2, prompt, 12)
    assert c_toks == a_toks and torch.equal(c_rows, a_rows)


@pytest.mark.parametrize("seed", [0, 7])
def test_sampled_streams_are_reproducible(seed):
    cfg, ckpt = shrunk_checkpoint(0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    prompt = synthetic_prompt(cfg.vocab, 16, seed=5)
    out = []
    for _ in range(2):
        eng.head.set_sampling_config(seed, 1.0, 0.95, 20)
        out.append([eng.prefill(prompt, chunk=8)] + eng.generate(max_new=10))
    assert out[0] == out[1]
