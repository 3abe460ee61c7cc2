"""The MTP draft layer and the sampled multi-row verify step against their fp32 CPU oracles (``mtp/reference.py``).

``tests/test_mtp_gpu.py`` checks that the emitted stream is the greedy stream, which holds for ANY draft, including a
broken one.  Here the draft path itself is pinned: the draft layer's K/V rows after a prefill, the first draft, and the
two chained drafts must be what the oracle computes from the target's hidden states; and the verifier's sampler at
temperature > 0 - per-row sampling with the position-keyed generator, prefix accept, commit, the poison matrix and the
forced commit counts replayed inside a captured graph - must match ``verify_reference`` word for word
(reference: nex_n2_5_pro/mtp/sampling_ref.py:30-143, tests/test_speculative_sampling_gpu.py).
"""

import pytest
import torch

from nexrt_b200.models.reference import RefModel, rms_norm, robust_prompt, synthetic_prompt
from nexrt_b200.mtp import MtpDraft
from nexrt_b200.mtp.reference import RefMtpDraft, verify_reference
from nexrt_b200.mtp.weights import random_mtp_checkpoint, shard_mtp
from nexrt_b200.runtime.control import Ctl, Status
from nexrt_b200.testing import gather_logits, make_engine, shrunk_checkpoint

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


@pytest.fixture(scope="module")
def setup():
    cfg, ckpt = shrunk_checkpoint(0)
    dev = torch.device("cuda", 0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    eng.head.enable_logits()
    mtp_ckpt = random_mtp_checkpoint(cfg, 7)
    mtp = MtpDraft(eng, shard_mtp(mtp_ckpt, cfg, 1, 0, dev, eng.head.w))
    return cfg, ckpt, mtp_ckpt, eng, mtp


def _near(logits, tok):
    return tok == int(logits.argmax()) or float(logits.max() - logits[tok]) < 0.05


def test_draft_layer_matches_the_oracle(setup):
    cfg, ckpt, mtp_ckpt, eng, mtp = setup
    ref, dref = RefModel(cfg, ckpt), RefMtpDraft(cfg, ckpt, mtp_ckpt)
    prompt, _ = robust_prompt(ref, cfg.vocab, 21, seeds=range(1, 9))
    ref.reset()
    hidden = [ref.step(t, return_hidden=True) for t in prompt]
    first_logits = ref.lm_head @ rms_norm(hidden[-1], ref.final_ln, cfg.rms_eps)
    first = mtp.prefill(prompt, chunk=8)
    assert _near(first_logits, first) and eng.status_max() == 0
    # draft-layer position p pairs the target's hidden row of p with the token of p + 1
    nxt = prompt[1:] + [first]
    for p, (h, t) in enumerate(zip(hidden, nxt)):
        logits, out = dref.step(h, t, p)
    want_k, want_v = dref.kv()
    L = len(prompt)
    assert rel_l2(mtp.attn.k_cache[:, :L].float().cpu(), want_k) < 2e-2
    assert rel_l2(mtp.attn.v_cache[:, :L].float().cpu(), want_v) < 2e-2
    draft1 = eng.read_ctl()["ids"][1]
    assert _near(logits, draft1), (draft1, int(logits.argmax()))
    # the two chained single-row passes: the draft layer's own output hidden, the previous draft as the token
    eng.ctx.begin_step()
    mtp.draft_phase()
    eng.step_end()
    torch.cuda.synchronize()
    ids = eng.read_ctl()["ids"]
    logits2, out2 = dref.step(out, draft1, L)
    assert _near(logits2, ids[2]), (ids[2], int(logits2.argmax()))
    logits3, _ = dref.step(out2, ids[2], L + 1)
    assert _near(logits3, ids[3]), (ids[3], int(logits3.argmax()))
    assert eng.status_max() == 0


@pytest.mark.parametrize("rows", [4, 8])
@pytest.mark.parametrize("seed,t,p,k", [(11, 0.8, 0.9, 10), (12, 1.2, 1.0, 28), (13, 0.0, 1.0, 1)])
def test_sampled_verify_matches_the_oracle(setup, rows, seed, t, p, k):
    cfg, ckpt, mtp_ckpt, eng, mtp = setup
    prompt = synthetic_prompt(cfg.vocab, 16, seed=30 + rows)
    eng.head.set_sampling_config(seed, t, p, k)
    first = eng.prefill(prompt, chunk=8)
    C = eng.read_ctl()["committed_len"]
    drafts = [int(x) for x in torch.randint(0, cfg.vocab, (rows - 1,), generator=torch.Generator().manual_seed(seed))]
    ids = [first] + drafts
    eng.set_rows(ids)
    eng.step(rows)
    logits = gather_logits(eng, rows)
    ctl = eng.read_ctl()
    want = verify_reference(list(logits), ids, C, seed, t, p, k)
    # the sampler's export buffer: kept ids, their probabilities and the sampled token of every row
    exp = eng.ctx.head_export[:rows].cpu()
    for j in range(rows):
        kept_ids, probs = want["kept"][j]
        n_kept = int(exp[j, 57])
        assert n_kept == len(kept_ids) or t == 0.0
        assert int(exp[j, 56]) in kept_ids
    # a row whose fp32 cumulative sum lands on the other side of a bucket edge than the float64 oracle picks a neighbour
    # token; everything after the first such row follows from the device's own choice, so the words are compared up to it
    target_dev = [int(exp[j, 56]) for j in range(rows)]
    again = verify_reference(list(logits), ids, C, seed, t, p, k)
    if target_dev == want["target"]:
        for key in ("commit_count", "accepted", "pending", "committed_len"):
            assert ctl[key] == want[key], (key, ctl[key], want[key])
        assert ctl["emitted"] == want["emitted"]
    else:
        assert sum(a != b for a, b in zip(target_dev, want["target"])) <= 1
    assert ctl["status"] == 0 and again["target"] == want["target"]
    eng.head.set_sampling_config(0, 0.0, 1.0, 1)


def test_poison_matrix_commits_nothing(setup):
    cfg, ckpt, mtp_ckpt, eng, mtp = setup
    prompt = synthetic_prompt(cfg.vocab, 16, seed=41)
    good = (5, 0.7, 0.9, 8)
    for poison in ("upstream", "bad_top_k", "nan_temperature"):
        eng.head.set_sampling_config(*good)
        first = eng.prefill(prompt, chunk=8)
        before = eng.read_ctl()["committed_len"]
        if poison == "upstream":
            eng.ctx.ctl[Ctl.STATUS] = int(Status.REDUCE_TIMEOUT)
        elif poison == "bad_top_k":
            eng.ctx.sampling[2] = 99
        else:
            eng.ctx.sampling[1] = (eng.ctx.sampling[1] & ~0xFFFFFFFF) | 0x7FC00000     # temperature bits := NaN
        eng.set_rows([first, 1, 2, 3])
        eng.step(4)
        ctl = eng.read_ctl()
        assert ctl["commit_count"] == 0 and ctl["committed_len"] == before and ctl["pending"] == -1, (poison, ctl)
        assert ctl["status"] != 0 and ctl["emitted"] == [-1] * 8
    eng.head.set_sampling_config(0, 0.0, 1.0, 1)


@pytest.mark.parametrize("rows", [4, 8])
def test_forced_commit_counts_replayed_in_a_graph(setup, rows):
    """The forced commit count lives in the control block, so one captured graph serves every count."""
    cfg, ckpt, mtp_ckpt, eng, mtp = setup
    eng.prefill(synthetic_prompt(cfg.vocab, 16, seed=43), chunk=8)
    g = eng.capture(rows)
    for n in range(1, rows + 1):
        before = eng.read_ctl()["committed_len"]
        eng.set_forced_commit(n)
        g.replay()
        torch.cuda.synchronize()
        ctl = eng.read_ctl()
        assert ctl["commit_count"] == n and ctl["committed_len"] == before + n and ctl["status"] == 0
    eng.set_forced_commit(0)
