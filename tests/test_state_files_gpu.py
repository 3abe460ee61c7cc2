"""Prefill-state files: a boundary saved by extract_state.save_state and installed by load_state into a
fresh engine continues with exactly the same tokens; decode_matrix's teacher-forced golden comparison
accepts the engine's own stream."""

import pytest
import torch

from nexrt_b200.decode_matrix import compare_with_golden
from nexrt_b200.extract_state import load_state, save_state, state_dir
from nexrt_b200.models.reference import synthetic_prompt
from nexrt_b200.testing import make_engine, shrunk_checkpoint

pytestmark = pytest.mark.gpu


def test_state_file_roundtrip_and_golden(tmp_path):
    cfg, ckpt = shrunk_checkpoint(0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    prompt = synthetic_prompt(cfg.vocab, 37, seed=31)
    first = eng.prefill(prompt, chunk=8)
    snap = eng._snapshot()
    golden = [first] + eng.generate(max_new=9)
    eng._restore(snap)
    out = state_dir(tmp_path, cfg.n_layers, len(prompt))
    path = save_state(eng, prompt, out, golden)
    assert path.name == "prefill_state_rank0.pt" and (out / "prefill_meta.pt").is_file() and (out / "golden.pt").is_file()
    meta = torch.load(out / "prefill_meta.pt", weights_only=False)
    assert meta["L"] == len(prompt) and meta["first_token"] == first and meta["prompt_ids"] == prompt

    fresh = make_engine(cfg, ckpt, max_rows=8)
    fresh.head.enable_logits()
    state = load_state(fresh, out)
    assert state["L"] == len(prompt) and fresh.read_ctl()["pending"] == first
    graph = fresh.capture(1)
    snap2 = fresh._snapshot()
    assert [first] + fresh.generate(graph, max_new=9) == golden
    fresh._restore(snap2)
    report = compare_with_golden(fresh, golden, steps=9, graph=graph)
    assert report["compared"] == 9 and not report["mismatches"]
    # a stream that is wrong somewhere is reported (unless the engine's own logits call it a near tie)
    fresh._restore(snap2)
    wrong = list(golden)
    wrong[4] = (wrong[4] + 1) % cfg.vocab
    bad = compare_with_golden(fresh, wrong, steps=9, graph=graph)
    assert bad["mismatches"] or bad["near_ties"]
    with pytest.raises(ValueError):
        state["tp"] = 2
        torch.save(state, out / "prefill_state_rank0.pt")
        load_state(fresh, out)
