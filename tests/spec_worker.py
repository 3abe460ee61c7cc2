"""Child process of tests/test_tp_gpu.py::test_speculative_drafts_tp2: the MTP draft layer and the DFlash block draft on a
tensor-parallel engine against their fp32 CPU oracles - draft K/V (this rank's kv heads), draft ids, and the same ids on
every rank."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nexrt_b200.dflash import DFlashBlock, shrunk_dflash_config  # noqa: E402
from nexrt_b200.dflash.reference import RefDFlashDraft  # noqa: E402
from nexrt_b200.dflash.weights import load_dflash_shard, random_dflash_checkpoint  # noqa: E402
from nexrt_b200.models.reference import RefModel, rms_norm, robust_prompt  # noqa: E402
from nexrt_b200.mtp import MtpDraft  # noqa: E402
from nexrt_b200.mtp.reference import RefMtpDraft  # noqa: E402
from nexrt_b200.mtp.weights import random_mtp_checkpoint, shard_mtp  # noqa: E402
from nexrt_b200.testing import make_engine, shrunk_checkpoint  # noqa: E402


def rel_l2(a, b):
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def near(logits, tok, tol=0.05):
    return tok == int(logits.argmax()) or float(logits.max() - logits[tok]) < tol


def same_on_every_rank(values, dev):
    t = torch.tensor(list(values), device=dev)
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t)
    return all(torch.equal(out[0], u) for u in out)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg, ckpt = shrunk_checkpoint(0)
    ref = RefModel(cfg, ckpt)
    prompt, _ = robust_prompt(ref, cfg.vocab, 21, n_new=8, seeds=range(1, 9))
    L = len(prompt)

    # ---- MTP ------------------------------------------------------------------------------------------------------
    eng = make_engine(cfg, ckpt, rank=rank, world=world, device=dev, max_rows=8)
    mtp_ckpt = random_mtp_checkpoint(cfg, 7)
    mtp = MtpDraft(eng, shard_mtp(mtp_ckpt, cfg, world, rank, dev, eng.head.w))
    dref = RefMtpDraft(cfg, ckpt, mtp_ckpt)
    ref.reset()
    hidden = [ref.step(t, return_hidden=True) for t in prompt]
    first_logits = ref.lm_head @ rms_norm(hidden[-1], ref.final_ln, cfg.rms_eps)
    first = mtp.prefill(prompt, chunk=8)
    assert near(first_logits, first) and eng.status_max() == 0
    for p, (h, t) in enumerate(zip(hidden, prompt[1:] + [first])):
        logits, out = dref.step(h, t, p)
    want_k, want_v = dref.kv()
    h0, nh = eng.spec.kv_head0, eng.spec.kv_heads
    assert rel_l2(mtp.attn.k_cache[:, :L].float().cpu(), want_k[h0 : h0 + nh]) < 2e-2
    assert rel_l2(mtp.attn.v_cache[:, :L].float().cpu(), want_v[h0 : h0 + nh]) < 2e-2
    eng.ctx.begin_step()
    mtp.draft_phase()
    eng.step_end()
    torch.cuda.synchronize()
    ids = eng.read_ctl()["ids"]
    assert near(logits, ids[1]), ("draft 1", ids[1], int(logits.argmax()))
    logits2, out2 = dref.step(out, ids[1], L)
    assert near(logits2, ids[2]), ("draft 2", ids[2], int(logits2.argmax()))
    logits3, _ = dref.step(out2, ids[2], L + 1)
    assert near(logits3, ids[3]), ("draft 3", ids[3], int(logits3.argmax()))
    assert same_on_every_rank(ids[:4], dev) and eng.status_max() == 0
    del mtp, eng

    # ---- DFlash ----------------------------------------------------------------------------------------------------
    eng = make_engine(cfg, ckpt, rank=rank, world=world, device=dev, max_rows=8)
    dc = shrunk_dflash_config(cfg)
    dckpt = random_dflash_checkpoint(dc, 11)
    block = DFlashBlock(eng, dc, load_dflash_shard(dckpt, dc, world, rank, dev))
    ref.tap_layers = tuple(dc.target_layer_ids)
    ref.reset()
    oracle = RefDFlashDraft(dc, dckpt, ref.embed, ref.lm_head)
    for p, t in enumerate(prompt):
        ref.step(t)
        oracle.context(p, ref.last_taps)
    first = block.prefill(prompt)
    kv_local = dc.n_kv_heads // world
    for l in range(dc.n_layers):
        want_k, want_v = oracle.kv(l, L)
        sl = slice(rank * kv_local, (rank + 1) * kv_local)
        assert rel_l2(block.k_cache[l][:, :L].float().cpu(), want_k[sl]) < 2e-2, l
        assert rel_l2(block.v_cache[l][:, :L].float().cpu(), want_v[sl]) < 2e-2, l
    eng.ctx.begin_step()
    block.context_phase()
    block.draft_phase()
    torch.cuda.synchronize()
    ids = eng.read_ctl()["ids"]
    _, want_logits = oracle.draft(first, L)
    assert ids[0] == first
    for j in range(1, 8):
        assert near(want_logits[j], ids[j], 0.02), ("proposal", j, ids[j], int(want_logits[j].argmax()))
    eng.step(8, end=False, begin=False)
    eng.step_end()
    torch.cuda.synchronize()
    assert same_on_every_rank(ids, dev) and eng.status_max() == 0
    dist.barrier()
    if rank == 0:
        print("SPEC_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
