"""MTP speculative decoding on one GPU (shrunk model, random-init draft layer): the emitted stream
is the plain greedy stream whatever the drafts are (reference tests/test_mtp_e2e_golden.py), perfect
drafts are accepted in full, and the forced-commit controls behave (test_speculative_sampling_gpu.py)."""

import pytest
import torch

from nexrt_b200.models.reference import RefModel, robust_prompt, synthetic_prompt
from nexrt_b200.mtp import MtpDraft, capture_round, generate_mtp
from nexrt_b200.mtp.weights import random_mtp_checkpoint, shard_mtp
from nexrt_b200.runtime.control import Ctl
from nexrt_b200.testing import make_engine, shrunk_checkpoint
from nexrt_b200.weights import shard_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup():
    cfg, ckpt = shrunk_checkpoint(0)
    dev = torch.device("cuda", 0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    head = shard_model(ckpt, cfg, 1, 0, dev)["head"]
    mtp = MtpDraft(eng, shard_mtp(random_mtp_checkpoint(cfg, 7), cfg, 1, 0, dev, eng.head.w))
    ref = RefModel(cfg, ckpt)
    return cfg, ref, eng, mtp


def _check_stream(got, toks_ref, logits_ref):
    for i, (a, b) in enumerate(zip(got, toks_ref)):
        if a != b:
            assert logits_ref[i].max() - logits_ref[i][a] < 0.05, (i, a, b)
            return
    assert len(got) == len(toks_ref)


def test_mtp_stream_equals_greedy_stream(setup):
    cfg, ref, eng, mtp = setup
    prompt = synthetic_prompt(cfg.vocab, 40, seed=11)
    ref.reset()
    toks_ref, logits_ref = ref.greedy(prompt, 13)
    first = mtp.prefill(prompt, chunk=8)
    g = capture_round(mtp)
    stats = {}
    out = generate_mtp(mtp, g, max_new=12, stats=stats)
    _check_stream([first] + out, toks_ref, logits_ref)
    assert eng.status_max() == 0 and stats["rounds"] >= 3 and 1.0 <= stats["accept_mean"] <= 4.0


def test_perfect_drafts_are_all_accepted(setup):
    cfg, ref, eng, mtp = setup
    # expert selection is discontinuous: compare arithmetics on a prompt whose routing margins are wide
    prompt, _ = robust_prompt(ref, cfg.vocab, 24, n_new=6, seeds=range(1, 17))
    toks_ref, _ = ref.greedy(prompt, 6)
    first = eng.prefill(prompt, chunk=8)
    assert first == toks_ref[0]
    eng.set_rows(toks_ref[0:4])            # pending token followed by the three true next tokens
    eng.step(4)
    ctl = eng.read_ctl()
    if ctl["accepted"] == 3:               # (a near-tie in the 4-row arithmetic may cut the prefix short)
        assert ctl["commit_count"] == 4 and ctl["emitted"][:4] == toks_ref[1:5] and ctl["pending"] == toks_ref[4]
    else:
        assert ctl["emitted"][: ctl["commit_count"]] == toks_ref[1 : 1 + ctl["commit_count"]]
    assert ctl["committed_len"] == len(prompt) + ctl["commit_count"] and ctl["status"] == 0


def test_wrong_drafts_commit_one_token(setup):
    cfg, ref, eng, mtp = setup
    prompt, _ = robust_prompt(ref, cfg.vocab, 16, n_new=3, seeds=range(1, 17))
    toks_ref, _ = ref.greedy(prompt, 3)
    first = eng.prefill(prompt, chunk=8)
    wrong = [(t + 1) % cfg.vocab for t in toks_ref[1:4]]
    eng.set_rows([first] + wrong)
    eng.step(4)
    ctl = eng.read_ctl()
    assert ctl["accepted"] == 0 and ctl["commit_count"] == 1 and ctl["emitted"][0] == toks_ref[1]
    assert ctl["emitted"][1:] == [-1] * 7


def test_forced_commit_and_seeded_schedule(setup):
    cfg, ref, eng, mtp = setup
    eng.prefill(synthetic_prompt(cfg.vocab, 16, seed=14), chunk=8)
    for n in (1, 2, 3, 4):
        before = eng.read_ctl()["committed_len"]
        eng.set_forced_commit(n)
        eng.step(4)
        ctl = eng.read_ctl()
        assert ctl["commit_count"] == n and ctl["committed_len"] == before + n
    eng.set_forced_commit(0, seed=1234, mean10=30)
    counts = []
    for _ in range(40):
        eng.step(4)
        counts.append(eng.read_ctl()["commit_count"])
    assert all(1 <= c <= 4 for c in counts) and 2.5 <= sum(counts) / len(counts) <= 3.5
    eng.set_forced_commit(0)


def test_m4_verify_view_drives_the_same_step(setup):
    """``M4Verify`` (the reference's verifier API, m4_verify.py:155-1227) is a view of the engine: load + run verify four
    rows, accept the true continuation, and the forced-commit property and schedule reach the control block."""
    from nexrt_b200.m4_verify import M4Verify, M4VerifyCp

    cfg, ref, eng, mtp = setup
    prompt, _ = robust_prompt(ref, cfg.vocab, 24, n_new=6, seeds=range(1, 17))
    toks_ref, _ = ref.greedy(prompt, 6)
    first = eng.prefill(prompt, chunk=8)
    v = M4Verify(eng)
    assert v.eng is eng and first == toks_ref[0]
    v.load(toks_ref[0:4])
    v.run(end=True, begin=True)
    ctl = eng.read_ctl()
    assert ctl["status"] == 0 and 1 <= ctl["commit_count"] <= 4
    assert ctl["emitted"][: ctl["commit_count"]] == toks_ref[1 : 1 + ctl["commit_count"]]
    assert ctl["committed_len"] == len(prompt) + ctl["commit_count"]
    before = ctl["committed_len"]
    v.forced_commit = 2
    assert v.forced_commit == 2
    v.run(end=True, begin=True)
    ctl = eng.read_ctl()
    assert ctl["commit_count"] == 2 and ctl["committed_len"] == before + 2
    v.set_forced_schedule(seed=7, mean_accept=3.0)
    counts = []
    for _ in range(20):
        v.run(end=True, begin=True)
        counts.append(eng.read_ctl()["commit_count"])
    assert all(1 <= c <= 4 for c in counts) and 2.0 <= sum(counts) / len(counts) <= 4.0
    v.forced_commit = 0
    with pytest.raises(ValueError):
        M4VerifyCp(eng)                  # a single-rank engine has no context-parallel arm


def test_upstream_status_fails_closed(setup):
    cfg, ref, eng, mtp = setup
    eng.prefill(synthetic_prompt(cfg.vocab, 16, seed=15), chunk=8)
    before = eng.read_ctl()["committed_len"]
    eng.ctx.ctl[Ctl.STATUS] = 1          # a failure latched by any earlier kernel (set on the host)
    eng.step(4)
    ctl = eng.read_ctl()
    assert ctl["commit_count"] == 0 and ctl["committed_len"] == before and ctl["pending"] == -1 and ctl["status"] != 0


def test_wide_prefill_feeds_the_draft_layer(setup):
    """Target prefilled in wide chunks, draft layer extended eight rows at a time on the chunks' hidden rows: the draft
    cache agrees with the one the 8-row prefill leaves (to the FP8 rounding of the wide path), and the rounds that follow
    emit what plain decode emits from the same prefill."""
    cfg, ref, eng, mtp = setup
    prompt = synthetic_prompt(cfg.vocab, 53, seed=13)
    mtp.prefill(prompt, chunk=8, wide=0)
    want_k = mtp.attn.k_cache[:, :52].float().clone()
    first = mtp.prefill(prompt, chunk=8, wide=16)
    assert eng.status_max() == 0 and any(key[0] == 16 for key in eng._wide)
    got_k = mtp.attn.k_cache[:, :52].float()
    assert float((got_k - want_k).norm() / want_k.norm()) < 0.3
    stats = {}
    out = generate_mtp(mtp, capture_round(mtp), max_new=10, stats=stats)
    assert eng.status_max() == 0 and len(out) == 10 and stats["rounds"] >= 3
    first_plain = eng.prefill(prompt, chunk=8, wide=16)
    plain = eng.generate(max_new=10)
    assert first_plain == first
    same = 0
    for a, b in zip(out, plain):       # a near tie between the 4-row and the 1-row arithmetic may end the common prefix early
        if a != b:
            break
        same += 1
    assert same >= 3, (out, plain)
