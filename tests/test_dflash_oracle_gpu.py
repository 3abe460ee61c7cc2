"""The DFlash block draft against its fp32 CPU oracle (``dflash/reference.py``): the context K/V the prefill leaves in
every draft layer, the eight-row block's logits and proposals ``ids[1..7]``, and the same again one round later, when the
context rows come from the features of the rows the verify step committed (sliding-window and full layers both).
``tests/test_dflash_gpu.py`` only checks that the emitted stream is the greedy stream, which any draft satisfies."""

import pytest
import torch

from nexrt_b200.dflash import DFlashBlock, shrunk_dflash_config
from nexrt_b200.dflash.reference import RefDFlashDraft
from nexrt_b200.dflash.weights import load_dflash_shard, random_dflash_checkpoint
from nexrt_b200.models.reference import RefModel, robust_prompt
from nexrt_b200.testing import make_engine, shrunk_checkpoint

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def _draft_on_device(block):
    """Context and draft phase of one round; returns (proposed ids[0..7], draft logits [8, vocab]) and leaves the verify to the caller."""
    eng = block.eng
    eng.ctx.begin_step()
    block.context_phase()
    block.draft_phase()
    torch.cuda.synchronize()
    return eng.read_ctl()["ids"], block.head.logits[:8].float().cpu()


def _check_block(ids, logits, want_logits, first):
    assert ids[0] == first
    for j in range(1, 8):
        assert rel_l2(logits[j], want_logits[j]) < 2e-2, (j, rel_l2(logits[j], want_logits[j]))
        assert ids[j] == int(want_logits[j].argmax()) or float(want_logits[j].max() - want_logits[j][ids[j]]) < 0.02, j


def test_dflash_draft_matches_the_oracle():
    cfg, ckpt = shrunk_checkpoint(0)
    dev = torch.device("cuda", 0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    dc = shrunk_dflash_config(cfg)
    dckpt = random_dflash_checkpoint(dc, 11)
    block = DFlashBlock(eng, dc, load_dflash_shard(dckpt, dc, 1, 0, dev))
    block.head.enable_logits()
    ref = RefModel(cfg, ckpt)
    prompt, _ = robust_prompt(ref, cfg.vocab, 21, n_new=8, seeds=range(1, 9))
    ref.tap_layers = tuple(dc.target_layer_ids)
    ref.reset()
    oracle = RefDFlashDraft(dc, dckpt, ref.embed, ref.lm_head)
    for p, t in enumerate(prompt):
        logits = ref.step(t)
        oracle.context(p, ref.last_taps)
    L = len(prompt)
    first = block.prefill(prompt)
    assert first == int(logits.argmax()) or float(logits.max() - logits[first]) < 0.05
    for l in range(dc.n_layers):
        want_k, want_v = oracle.kv(l, L)
        assert rel_l2(block.k_cache[l][:, :L].float().cpu(), want_k) < 2e-2, l
        assert rel_l2(block.v_cache[l][:, :L].float().cpu(), want_v) < 2e-2, l
    # first draft round: the block at base position L
    ids, dev_logits = _draft_on_device(block)
    _, want_logits = oracle.draft(first, L)
    _check_block(ids, dev_logits, want_logits, first)
    for l in range(dc.n_layers):      # the block's own rows were published at L .. L + 7
        want_k, _ = oracle.kv(l, L + 8)
        assert rel_l2(block.k_cache[l][:, L : L + 8].float().cpu(), want_k[:, L:]) < 2e-2, l
    eng.step(8, end=False, begin=False)
    eng.step_end()
    torch.cuda.synchronize()
    ctl = eng.read_ctl()
    n = ctl["commit_count"]
    assert 1 <= n <= 8 and ctl["status"] == 0
    # the verify step consumed ids[0 .. n-1] at positions L .. L + n - 1: their features become context rows
    for j in range(n):
        ref.step(ids[j])
        oracle.context(L + j, ref.last_taps)
    # second draft round
    ids2, dev_logits2 = _draft_on_device(block)
    _, want2 = oracle.draft(ctl["pending"], L + n)
    _check_block(ids2, dev_logits2, want2, ctl["pending"])
    for l in range(dc.n_layers):
        want_k, want_v = oracle.kv(l, L + n)
        assert rel_l2(block.k_cache[l][:, L : L + n].float().cpu(), want_k[:, L:]) < 2e-2, l
        assert rel_l2(block.v_cache[l][:, L : L + n].float().cpu(), want_v[:, L:]) < 2e-2, l
    eng.step(8, end=False, begin=False)
    eng.step_end()
    torch.cuda.synchronize()
    assert eng.status_max() == 0
