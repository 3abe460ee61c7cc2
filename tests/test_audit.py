"""Guard bands and the pointer-disjointness audit (``runtime/audit.py``): on CPU tensors here, on a real engine below
(GPU): 1-, 4-, 5- and 8-row steps and a prefill leave every guard band of the context's scratch intact, and no two
buffers the kernels are launched on overlap."""

import os

import pytest
import torch

from nexrt_b200.runtime.audit import GUARD_BYTES, engine_tensors, guarded_zeros, named_tensors, overlaps, violated


def test_guard_bands_catch_a_write_past_the_end():
    reg = []
    a = guarded_zeros(reg, (3, 5), torch.float32, "cpu")
    b = guarded_zeros(reg, (7,), torch.int32, "cpu")
    assert a.shape == (3, 5) and a.dtype == torch.float32 and float(a.abs().sum()) == 0 and b.numel() == 7
    assert a.data_ptr() % 16 == 0 and violated(reg) == []
    a.fill_(1.0)
    b.fill_(-1)
    assert violated(reg) == []                      # writing the data is fine
    arena, nbytes = reg[0]
    arena[GUARD_BYTES + nbytes] = 0                 # one byte past the end of `a`: inside the padding
    assert violated(reg) == [0]
    arena[GUARD_BYTES + nbytes] = 0xA5
    reg[1][0][GUARD_BYTES - 1] = 7                  # one byte before `b`
    assert violated(reg) == [1]


def test_overlap_audit_ignores_views_and_reports_foreign_overlap():
    base = torch.zeros(64)
    holder = type("H", (), {})()
    holder.a, holder.view, holder.other = base, base[8:16], torch.zeros(16)
    holder.nested = {"w": [torch.zeros(4), base[:4]]}
    names = named_tensors(holder, "h")
    assert {"h.a", "h.view", "h.other", "h.nested.w.0", "h.nested.w.1"} <= set(names)
    assert overlaps(names) == []
    # two tensors over the same bytes that do not share a storage object: built from one buffer through the array interface
    import numpy as np

    raw = np.zeros(64, dtype=np.float32)
    t1, t2 = torch.from_numpy(raw), torch.from_numpy(raw[4:12])
    if t1.untyped_storage().data_ptr() != t2.untyped_storage().data_ptr():
        assert overlaps({"x": t1, "y": t2}) == [("x", "y")]


@pytest.mark.gpu
def test_engine_steps_leave_guards_intact_and_buffers_disjoint(monkeypatch):
    from nexrt_b200.models.reference import synthetic_prompt
    from nexrt_b200.testing import make_engine, shrunk_checkpoint

    monkeypatch.setenv("NEXRT_CANARY", "1")
    cfg, ckpt = shrunk_checkpoint(0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    assert eng.ctx.canaries_violated() == []
    prompt = synthetic_prompt(cfg.vocab, 29, seed=4)
    eng.prefill(prompt, chunk=8)                    # 8, 8, 8, 5 rows
    for rows in (1, 4, 7):
        eng.set_rows(prompt[:rows])
        eng.set_forced_commit(rows)
        eng.step(rows)
    eng.set_forced_commit(0)
    eng.generate(max_new=3)
    assert eng.read_ctl()["status"] == 0
    assert eng.ctx.canaries_violated() == []
    assert overlaps(engine_tensors(eng)) == []
