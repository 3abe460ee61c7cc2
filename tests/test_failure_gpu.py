"""Failure detection without faulting the GPU: a peer that never sends makes the bounded waits of the
fused reduce kernels run out; the step must fail closed (status latched, nothing committed, token -1),
return promptly, and leave the context usable.  Device-side fault injection is not part of this
framework; the failure is made on the host."""

import time

import pytest
import torch

from nexrt_b200.models.reference import synthetic_prompt
from nexrt_b200.runtime.control import Ctl, Status
from nexrt_b200.testing import attach_silent_peer, make_engine, shrunk_checkpoint

pytestmark = pytest.mark.gpu


def test_silent_peer_times_out_and_fails_closed():
    cfg, ckpt = shrunk_checkpoint(0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    prompt = synthetic_prompt(cfg.vocab, 16, seed=2)
    eng.prefill(prompt, chunk=8)
    before = eng.read_ctl()
    assert before["status"] == 0 and before["committed_len"] == 16
    attach_silent_peer(eng, budget_ms=50.0)
    t0 = time.time()
    eng.step(1)
    torch.cuda.synchronize()
    elapsed = time.time() - t0
    after = eng.read_ctl()
    assert after["status"] == Status.REDUCE_TIMEOUT
    assert after["committed_len"] == before["committed_len"] and after["commit_count"] == 0 and after["pending"] == -1
    # the first wait spends its budget, every later wait sees the latched failure and gives up at once
    assert elapsed < 5.0, elapsed
    # the CUDA context is intact: a healthy engine on the same device still decodes
    other = make_engine(cfg, ckpt, max_rows=8)
    first = other.prefill(prompt, chunk=8)
    assert first >= 0 and other.read_ctl()["status"] == 0


def test_generate_raises_on_a_failed_step_and_serving_classifies_it():
    from nexrt_b200.serve.serve_control import is_fatal_backend_error

    cfg, ckpt = shrunk_checkpoint(0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    eng.prefill(synthetic_prompt(cfg.vocab, 8, seed=3), chunk=8)
    attach_silent_peer(eng, budget_ms=20.0)      # before the capture: a graph keeps the channel it was captured with
    with pytest.raises(RuntimeError) as info:
        eng.generate(max_new=4)
    assert "status" in str(info.value) and not is_fatal_backend_error(info.value)   # recoverable: reset the request, keep serving
    assert int(eng.ctx.ctl[Ctl.STATUS]) == Status.REDUCE_TIMEOUT


def test_failed_eight_row_unit_runs_again_after_reset_unit():
    """An 8-row verify unit that failed (its peer stayed silent) is re-executed from the same base after ``reset_unit``:
    the state rings are position indexed with a spare slot, so the second run reads what the first one read
    (reference tests/test_m8_state_units.py, m8_verify.py:722-741)."""
    from nexrt_b200.m8_verify import M8Verify
    from nexrt_b200.models.reference import RefModel, robust_prompt
    from nexrt_b200.testing import detach_silent_peer, gather_logits

    cfg, ckpt = shrunk_checkpoint(0)
    ref = RefModel(cfg, ckpt)
    prompt, _ = robust_prompt(ref, cfg.vocab, 24, seeds=range(1, 9))
    ref.reset()
    want = torch.stack([ref.step(t) for t in prompt])[16:]
    eng = make_engine(cfg, ckpt, max_rows=8)
    eng.head.enable_logits()
    eng.prefill(prompt[:16], chunk=8)
    unit = M8Verify(eng)
    attach_silent_peer(eng, budget_ms=30.0)
    unit.seed(prompt[16:24])
    eng.set_forced_commit(8)
    unit.run(begin=True, end=True)
    torch.cuda.synchronize()
    failed = eng.read_ctl()
    assert failed["status"] == Status.REDUCE_TIMEOUT and failed["committed_len"] == 16 and failed["commit_count"] == 0
    detach_silent_peer(eng)
    unit.reset_unit()
    unit.seed(prompt[16:24])            # the failed commit cleared ids[0]
    unit.run(begin=True, end=True)
    got = gather_logits(eng, 8)
    ctl = eng.read_ctl()
    assert ctl["status"] == 0 and ctl["committed_len"] == 24 and ctl["commit_count"] == 8
    err = float((got - want).norm() / want.norm())
    assert err < 2e-2, err
