"""DFlash speculative decoding on one GPU: shrunk target + small random draft.  The emitted stream
must equal the greedy stream whatever the proposals are; the dense projection kernel is checked
against fp32 PyTorch."""

import pytest
import torch

from nexrt_b200.dflash import DFlashBlock, capture_request, generate_dflash, shrunk_dflash_config
from nexrt_b200.dflash.weights import load_dflash_shard, random_dflash_checkpoint
from nexrt_b200.m8_verify import M8Verify
from nexrt_b200.models.reference import RefModel, synthetic_prompt
from nexrt_b200.ops import lib as L
from nexrt_b200.testing import make_engine, shrunk_checkpoint

pytestmark = pytest.mark.gpu


def test_dense_bf16_kernel_matches_fp32():
    lib = L.load()
    from nexrt_b200.parallel.channel import LLChannel

    dev = torch.device("cuda", 0)
    ch = LLChannel(dev, 1, 0, 8 * 1024)
    g = torch.Generator(device="cuda").manual_seed(3)
    for (M, R, K) in [(1, 256, 1024), (8, 768, 1024), (5, 1024, 512)]:
        w = (torch.randn(R, K, generator=g, device=dev) * 0.05).to(torch.bfloat16)
        x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
        gamma = 1.0 + 0.1 * torch.randn(K, generator=g, device=dev)
        out = torch.zeros(M, R, device=dev)
        L.check(lib.nexrt_dense_bf16(x.data_ptr(), gamma.data_ptr(), w.data_ptr(), out.data_ptr(), None, R, K, M, 0, 0, 0, 1e-6, ch.ref, 0,
                                     torch.cuda.current_stream().cuda_stream), "dense")
        xf = x.float()
        xn = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma
        want = xn @ w.float().T
        torch.cuda.synchronize()
        assert float((out - want).norm() / want.norm()) < 1e-3
        # SwiGLU input, residual output
        gu = torch.randn(M, 2 * K, generator=g, device=dev)
        xres = torch.randn(M, R, generator=g, device=dev).to(torch.bfloat16)
        want2 = xres.float() + (torch.nn.functional.silu(gu[:, :K]) * gu[:, K:]) @ w.float().T
        L.check(lib.nexrt_dense_bf16(gu.data_ptr(), None, w.data_ptr(), None, xres.data_ptr(), R, K, M, 2, 1, 0, 1e-6, ch.ref, 0,
                                     torch.cuda.current_stream().cuda_stream), "dense")
        torch.cuda.synchronize()
        assert float((xres.float() - want2).norm() / want2.norm()) < 1e-2


def test_dflash_stream_equals_greedy_stream():
    cfg, ckpt = shrunk_checkpoint(0)
    dev = torch.device("cuda", 0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    dc = shrunk_dflash_config(cfg)
    block = DFlashBlock(eng, dc, load_dflash_shard(random_dflash_checkpoint(dc, 11), dc, 1, 0, dev))
    assert M8Verify(eng).eng is eng
    prompt = synthetic_prompt(cfg.vocab, 40, seed=21)
    ref = RefModel(cfg, ckpt)
    toks_ref, logits_ref = ref.greedy(prompt, 11)
    first = block.prefill(prompt)
    g = capture_request(block)
    stats = {}
    out = [first] + generate_dflash(block, g, max_new=10, stats=stats)
    for i, (a, b) in enumerate(zip(out, toks_ref)):
        if a != b:
            assert logits_ref[i].max() - logits_ref[i][a] < 0.05, (i, a, b)
            break
    else:
        assert len(out) == len(toks_ref)
    assert eng.status_max() == 0 and stats["rounds"] >= 1


def test_wide_prefill_fills_the_context_caches():
    """Target prefilled in wide chunks that also record the feature taps; the draft's context phase follows eight rows at
    a time.  The context K/V agree with what the 8-row prefill leaves (to the FP8 rounding of the wide path) and the
    rounds that follow emit what plain decode emits from the same prefill."""
    cfg, ckpt = shrunk_checkpoint(0)
    dev = torch.device("cuda", 0)
    eng = make_engine(cfg, ckpt, max_rows=8)
    dc = shrunk_dflash_config(cfg)
    block = DFlashBlock(eng, dc, load_dflash_shard(random_dflash_checkpoint(dc, 11), dc, 1, 0, dev))
    prompt = synthetic_prompt(cfg.vocab, 53, seed=23)
    block.prefill(prompt, wide=0)
    want_k = block.k_cache[0][:, :48].float().clone()
    first = block.prefill(prompt, wide=16)
    assert eng.status_max() == 0 and len(eng._wide) == 1
    got_k = block.k_cache[0][:, :48].float()
    assert float((got_k - want_k).norm() / want_k.norm()) < 0.3
    out = generate_dflash(block, capture_request(block), max_new=10, stats={})
    assert eng.status_max() == 0 and len(out) >= 10
    plain_first = eng.prefill(prompt, chunk=8, wide=16)
    state = eng.export_state()
    plain = eng.generate(max_new=10)
    assert plain_first == first
    same = 0
    for a, b in zip(out, plain):
        if a != b:
            break
        same += 1
    if same < len(plain):
        # the 8-row and the 1-row arithmetic may part ways only at a near tie: replay the plain decode up to that step with
        # the logits kept and look at the gap between the two candidates
        eng.head.enable_logits()
        eng.load_prefill(state)
        for _ in range(same + 1):
            eng.step(1)
        gap = eng.logit_gap(out[same], plain[same])
        assert gap is not None and gap < 0.05, (same, gap, out, plain)
