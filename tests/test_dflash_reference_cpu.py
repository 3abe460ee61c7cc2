"""The CPU oracle of the DFlash draft checks itself (no GPU): the sliding window really hides old context rows, a missing
context row is an error rather than a silent zero, the block's rows land in the caches at their positions, and the
target oracle's feature taps have the draft's input width."""

from dataclasses import replace

import pytest
import torch

from nexrt_b200.dflash import shrunk_dflash_config
from nexrt_b200.dflash.reference import RefDFlashDraft
from nexrt_b200.dflash.weights import random_dflash_checkpoint
from nexrt_b200.models.reference import RefModel
from nexrt_b200.testing import shrunk_checkpoint


@pytest.fixture(scope="module")
def setup():
    cfg, ckpt = shrunk_checkpoint(0)
    ref = RefModel(cfg, ckpt)
    return cfg, ref


def _fill(oracle, ref, dc, tokens):
    ref.tap_layers = tuple(dc.target_layer_ids)
    ref.reset()
    for p, t in enumerate(tokens):
        ref.step(t)
        oracle.context(p, ref.last_taps)


def test_taps_and_block_rows(setup):
    cfg, ref = setup
    dc = shrunk_dflash_config(cfg)
    o = RefDFlashDraft(dc, random_dflash_checkpoint(dc, 11), ref.embed, ref.lm_head)
    _fill(o, ref, dc, [5, 6, 7, 8, 9, 10])
    assert ref.last_taps.shape == (dc.n_taps * cfg.hidden,)
    ids, logits = o.draft(11, 6)
    assert len(ids) == 8 and logits.shape == (8, cfg.vocab) and torch.isfinite(logits).all()
    k, v = o.kv(0, 14)
    assert k.shape == (dc.n_kv_heads, 14, dc.head_dim) and v.shape == k.shape
    again, logits2 = o.draft(11, 6)
    assert again == ids and torch.equal(logits, logits2)


def test_sliding_window_hides_old_rows_and_missing_rows_raise(setup):
    cfg, ref = setup
    dc = replace(shrunk_dflash_config(cfg), layer_types=("sliding", "sliding"), sliding_window=12)
    ck = random_dflash_checkpoint(dc, 11)
    tokens = list(range(20, 30))
    a = RefDFlashDraft(dc, ck, ref.embed, ref.lm_head)
    _fill(a, ref, dc, tokens)
    _, base_logits = a.draft(3, 10)            # keys 6 .. 17: positions 0 .. 5 are outside every layer's window
    for l in range(dc.n_layers):
        a.k[l][2] = a.k[l][2] + 1.0
    _, moved = a.draft(3, 10)
    assert torch.equal(base_logits, moved)
    for l in range(dc.n_layers):
        a.k[l][8] = a.k[l][8] + 1.0            # inside the window: the logits move
    _, moved = a.draft(3, 10)
    assert not torch.equal(base_logits, moved)
    del a.k[0][7]
    with pytest.raises(KeyError):
        a.draft(3, 10)
