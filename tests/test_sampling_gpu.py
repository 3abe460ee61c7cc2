"""Device sampler against the float64 CPU oracle: full-vocabulary sampler kernel over a matrix of
temperature / top-p / top-k / seed / position, the distributed head of the engine, and the poison
matrix (bad configuration, non-finite logits) that must latch a status instead of emitting a token."""

import itertools

import pytest
import torch

from nexrt_b200.models.reference import synthetic_prompt
from nexrt_b200.ops.lib import check, load, ptr
from nexrt_b200.runtime.control import CTL_WORDS, Ctl, Status
from nexrt_b200.sampling import sample_reference, sampling_words
from nexrt_b200.testing import gather_logits, make_engine, shrunk_checkpoint

pytestmark = pytest.mark.gpu


def _sample(logits, seed, pos, t, p, k, raw_words=None):
    dev = logits.device
    ctl = torch.zeros(CTL_WORDS, dtype=torch.int32, device=dev)
    words = torch.tensor(raw_words if raw_words is not None else sampling_words(seed, t, p, k), dtype=torch.int64, device=dev)
    check(load().nexrt_sample_logits(ptr(logits), ptr(words), ptr(ctl), logits.numel(), pos, torch.cuda.current_stream().cuda_stream), "sample")
    torch.cuda.synchronize()
    w = ctl.tolist()
    return w[Ctl.PENDING], w[Ctl.STATUS]


@pytest.mark.parametrize("t,p,k", list(itertools.product([0.0, 0.6, 1.3], [0.5, 0.95, 1.0], [1, 5, 20, 28])))
def test_sampler_kernel_matches_oracle(t, p, k):
    g = torch.Generator(device="cuda").manual_seed(int(t * 10) * 100 + k)
    logits = torch.randn(5000, device="cuda", generator=g) * 3
    mismatches = 0
    for seed, pos in [(0, 0), (1, 17), ((1 << 64) - 1, 123456), (0xDEADBEEF12345678, 4096)]:
        tok, status = _sample(logits, seed, pos, t, p, k)
        want, kept, probs = sample_reference(logits.cpu().numpy(), seed, pos, t, p, k)
        assert status == 0 and tok in kept
        mismatches += tok != want       # fp32 vs float64 cumulative sums may differ exactly at a bucket edge
    assert mismatches <= 1


def test_ties_go_to_the_lowest_token_id():
    logits = torch.zeros(1000, device="cuda")
    logits[[700, 30, 512]] = 5.0
    assert _sample(logits, 0, 0, 0.0, 1.0, 1) == (30, 0)


def test_poison_matrix_latches_status():
    logits = torch.randn(1000, device="cuda")
    good = sampling_words(0, 0.6, 0.95, 20)
    for words in ([good[0], good[1], 0] + [0] * 5, [good[0], good[1], 29] + [0] * 5, [good[0], good[1], -3] + [0] * 5):
        tok, status = _sample(logits, 0, 0, 0, 0, 0, raw_words=words)
        assert tok == -1 and status == Status.BAD_CONFIG
    bad = logits.clone()
    bad[5] = float("nan")
    bad[6] = float("inf")
    tok, status = _sample(bad, 0, 0, 0.6, 0.95, 20)
    assert tok == -1 and status == Status.NON_FINITE


def test_engine_head_samples_like_the_oracle_on_its_own_logits():
    cfg, ckpt = shrunk_checkpoint(0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    eng.head.enable_logits()
    prompt = synthetic_prompt(cfg.vocab, 12, seed=9)
    hits = 0
    cases = [(3, 0.8, 0.9, 10), (4, 1.0, 1.0, 28), (5, 0.3, 0.5, 4), (6, 0.0, 1.0, 1)]
    for seed, t, p, k in cases:
        eng.head.set_sampling_config(seed, t, p, k)
        tok = eng.prefill(prompt, chunk=8)
        logits = gather_logits(eng, 8)[(len(prompt) - 1) % 8]      # row of the last prompt token in the last chunk
        want, kept, _ = sample_reference(logits.numpy(), seed, len(prompt) - 1, t, p, k)
        assert tok in kept and eng.read_ctl()["status"] == 0
        hits += tok == want
    assert hits >= len(cases) - 1
