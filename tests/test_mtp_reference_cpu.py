"""The CPU oracles of the MTP path check themselves on hand-made vectors (no GPU): prefix accept, forced commit,
fail-closed words, position-keyed sampling that does not depend on the row count, and a draft-layer pass whose KV rows
are overwritten when an earlier position is replayed (reference: nex_n2_5_pro/mtp/sampling_ref.py:30-143)."""

import torch

from nexrt_b200.mtp.reference import RefMtpDraft, verify_reference
from nexrt_b200.mtp.weights import random_mtp_checkpoint
from nexrt_b200.testing import shrunk_checkpoint


def _rows(winners, vocab=32):
    out = []
    for w in winners:
        l = torch.zeros(vocab)
        l[w] = 5.0
        out.append(l)
    return out


def test_greedy_prefix_accept_and_commit_words():
    # targets 7, 9, 4, 2; drafts 7, 9, 3: two accepted, the third row's target is the bonus token
    r = verify_reference(_rows([7, 9, 4, 2]), [1, 7, 9, 3], 100, 0, 0.0, 1.0, 1)
    assert r["accepted"] == 2 and r["commit_count"] == 3 and r["pending"] == 4 and r["committed_len"] == 103
    assert r["emitted"] == [7, 9, 4, -1, -1, -1, -1, -1] and r["status"] == 0
    # a hole in the prefix stops the accept even if a later draft matches
    r = verify_reference(_rows([7, 9, 4, 2]), [1, 0, 9, 4], 100, 0, 0.0, 1.0, 1)
    assert r["accepted"] == 0 and r["commit_count"] == 1 and r["pending"] == 7


def test_forced_commit_and_upstream_failure():
    r = verify_reference(_rows([7, 9, 4, 2]), [1, 0, 0, 0], 10, 0, 0.0, 1.0, 1, forced_commit=3)
    assert r["commit_count"] == 3 and r["emitted"][:3] == [0, 0, 4] and r["committed_len"] == 13
    r = verify_reference(_rows([7, 9, 4, 2]), [1, 7, 9, 4], 10, 0, 0.0, 1.0, 1, upstream_status=4)
    assert r["commit_count"] == 0 and r["pending"] == -1 and r["committed_len"] == 10 and r["emitted"] == [-1] * 8 and r["status"] == 4


def test_eos_stop_position():
    r = verify_reference(_rows([7, 9, 4, 2]), [1, 7, 9, 4], 10, 0, 0.0, 1.0, 1, eos=9)
    assert r["stop_pos"] == 1 and r["commit_count"] == 4


def test_sampled_rows_do_not_depend_on_the_row_count():
    g = torch.Generator().manual_seed(3)
    rows = [torch.randn(64, generator=g) * 3 for _ in range(8)]
    ids = [1] + [0] * 7
    r8 = verify_reference(rows, ids, 50, 17, 0.9, 0.95, 12)
    r4 = verify_reference(rows[:4], ids[:4], 50, 17, 0.9, 0.95, 12)
    assert r8["target"][:4] == r4["target"]
    # the same logits at another position draw another uniform: over eight rows at least one token moves
    moved = verify_reference(rows, ids, 51, 17, 0.9, 0.95, 12)
    assert moved["target"] != r8["target"]


def test_draft_layer_replay_overwrites_speculative_rows():
    cfg, ckpt = shrunk_checkpoint(0)
    d = RefMtpDraft(cfg, ckpt, random_mtp_checkpoint(cfg, 7))
    g = torch.Generator().manual_seed(1)
    h = [torch.randn(cfg.hidden, generator=g).to(torch.bfloat16) for _ in range(3)]
    for p in range(3):
        logits, out = d.step(h[p], 5 + p, p)
    assert logits.shape == (cfg.vocab,) and out.dtype == torch.bfloat16 and torch.isfinite(logits).all()
    k3, _ = d.kv()
    assert k3.shape == (cfg.n_kv_heads, 3, cfg.head_dim)
    # replay position 1 with another token: rows 1.. are dropped and rewritten, row 0 is untouched
    d.step(h[1], 99, 1)
    k2, _ = d.kv()
    assert k2.shape[1] == 2 and torch.equal(k2[:, 0], k3[:, 0]) and not torch.equal(k2[:, 1], k3[:, 1])
    logits_b, _ = d.step(h[1], 6, 1)
    d2 = RefMtpDraft(cfg, ckpt, random_mtp_checkpoint(cfg, 7))
    d2.step(h[0], 5, 0)
    logits_c, _ = d2.step(h[1], 6, 1)
    assert torch.equal(logits_b, logits_c)
