"""Child process of the multi-GPU tests: one rank of a tensor-parallel engine over the shrunk
model, checked against the fp32 CPU oracle.  Launched by torchrun from test_tp_gpu.py."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nexrt_b200.models.reference import RefModel, robust_prompt, synthetic_prompt  # noqa: E402
from nexrt_b200.testing import make_engine, oracle_state, shard_oracle_state, shrunk_checkpoint  # noqa: E402


def rel_l2(a, b):
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg, ckpt = shrunk_checkpoint(0, tp8=os.environ.get("NEXRT_TEST_GEOMETRY") == "tp8")
    ref = RefModel(cfg, ckpt)
    eng = make_engine(cfg, ckpt, rank=rank, world=world, device=dev, max_rows=8)
    eng.head.enable_logits()
    V = cfg.vocab // world
    sl = slice(rank * V, (rank + 1) * V)
    print(f"[rank {rank}] symm={eng.ctx.channel.buf.backend} multicast={eng.ctx.channel.multicast}", flush=True)

    # single-row steps
    prompt, _ = robust_prompt(ref, cfg.vocab, 12)
    ref.reset()
    eng.reset(first_token=prompt[0])
    for tok in prompt:
        eng.set_rows([tok])
        eng.set_forced_commit(1)
        eng.step(1)
        torch.cuda.synchronize()
        got = eng.head.logits[0].float().cpu()
        want = ref.step(tok)[sl]
        assert rel_l2(got, want) < 2e-2, rel_l2(got, want)
    assert eng.status_max() == 0
    # the residual stream is bitwise identical on every rank
    xs = [torch.empty_like(eng.ctx.x) for _ in range(world)]
    dist.all_gather(xs, eng.ctx.x)
    assert all(torch.equal(xs[0].view(torch.int16), t.view(torch.int16)) for t in xs)

    # multi-row steps
    for rows in (4, 8):
        p2, _ = robust_prompt(ref, cfg.vocab, 2 * rows, seeds=range(50, 90))
        ref.reset()
        want = torch.stack([ref.step(t) for t in p2])[:, sl]
        eng.reset(first_token=p2[0])
        got = []
        for i in range(0, len(p2), rows):
            eng.set_rows(p2[i : i + rows])
            eng.set_forced_commit(rows)
            eng.step(rows)
            torch.cuda.synchronize()
            got.append(eng.head.logits[:rows].float().cpu())
        err = rel_l2(torch.cat(got), want)
        per_row = [round(rel_l2(a, b), 4) for a, b in zip(torch.cat(got), want)]
        assert err < 2e-2, (rows, err, per_row)

    # prefill + captured-graph generate: every rank emits the same stream, equal to the oracle's
    prompt, _ = robust_prompt(ref, cfg.vocab, 32, n_new=8, seeds=range(100, 140))
    ref.reset()
    toks_ref, logits_ref = ref.greedy(prompt, 8)
    first = eng.prefill(prompt, chunk=8)
    out = [first] + eng.generate(max_new=7)
    t = torch.tensor(out, device=dev)
    allt = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(allt, t)
    assert all(torch.equal(allt[0], u) for u in allt), allt
    for i, (a, b) in enumerate(zip(out, toks_ref)):
        if a != b:
            assert logits_ref[i].max() - logits_ref[i][a] < 0.05, (i, a, b)
            break
    assert eng.status_max() == 0

    # wide prefill chunks (tcgen05 GEMM per projection, all-reduce of the chunk's partial sums) against the 8-row steps
    long_prompt = synthetic_prompt(cfg.vocab, 53, seed=9)
    eng.prefill(long_prompt, chunk=8, wide=0)
    want_state = eng.export_state()
    first_w = eng.prefill(long_prompt, chunk=8, wide=16)          # default: the exact three-term activation split
    got_state = eng.export_state()
    assert eng.status_max() == 0 and got_state["L"] == 53 and eng.wide_path(16).P == 3
    for idx, st in want_state["layers"].items():
        for key, w_ in st.items():
            if key != "kind":
                # an order of magnitude under a lost row or block; a routing near tie of this arbitrary prompt may still turn
                assert rel_l2(got_state["layers"][idx][key].float(), w_.float()) < 0.1, (idx, key, rel_l2(got_state["layers"][idx][key].float(), w_.float()))
    t = torch.tensor([first_w], device=dev)
    allt = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(allt, t)
    assert all(torch.equal(allt[0], u) for u in allt), allt
    assert len(eng.generate(max_new=4)) == 4 and eng.status_max() == 0

    # the wide path with the exact activation split against the exact CPU oracle at the tolerance of the step kernels, on a
    # prompt that stays clear of routing near ties
    xprompt, _ = robust_prompt(ref, cfg.vocab, 53, seeds=range(1, 9))
    ref.reset()
    ref.prefill(xprompt)
    want_x = shard_oracle_state(oracle_state(ref), cfg, eng.spec)
    eng.prefill(xprompt, chunk=8, wide=16)
    got_x = eng.export_state()
    assert eng.status_max() == 0 and got_x["L"] == 53
    for idx, st in want_x.items():
        for key, w_ in st.items():
            have = got_x["layers"][idx][key].float().cpu()
            assert rel_l2(have, w_.float()) < 2e-2, ("wide, three terms, vs exact oracle", idx, key, rel_l2(have, w_.float()))

    # the wide path with ONE activation term against the CPU oracle with the SAME arithmetic (one e4m3 plane per FP8
    # projection input), held to the tolerance of the step kernels on this rank's shard of every layer's state: a lost block
    # of the chunk all-reduce, a wrong row of an attention sub-step or a mis-masked expert shows as an error of order one
    ref8 = RefModel(cfg, ckpt, fp8_activations=True)
    wprompt, _ = robust_prompt(ref8, cfg.vocab, 53, seeds=range(1, 9))
    ref8.reset()
    ref8.prefill(wprompt)
    want_w = shard_oracle_state(oracle_state(ref8), cfg, eng.spec)
    eng.wide_terms = 1
    eng.prefill(wprompt, chunk=8, wide=16)
    got_w = eng.export_state()
    assert eng.status_max() == 0 and got_w["L"] == 53
    n_wide = (53 - 1) // 16 * 16
    for idx, st in want_w.items():
        for key, w_ in st.items():
            have = got_w["layers"][idx][key].float().cpu()
            assert rel_l2(have, w_.float()) < 4e-2, ("wide vs matched oracle", idx, key, rel_l2(have, w_.float()))
            if key in ("k_cache", "v_cache"):
                per_pos = (have - w_.float()).norm(dim=-1) / w_.float().norm(dim=-1).clamp_min(1e-6)
                assert float(per_pos[:, :n_wide].max()) < 0.1, (idx, key, float(per_pos[:, :n_wide].max()))
    dist.barrier()
    if rank == 0:
        print("TP_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
