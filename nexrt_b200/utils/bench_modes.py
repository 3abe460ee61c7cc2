"""Round-time benchmark of the other decode modes: MTP (4-row verify, forced mean acceptance 3.0), DFlash
(8-row verify, forced mean acceptance 5.0), and batch-1 decode at long context with or without
context-parallel attention.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 -m nexrt_b200.utils.bench_modes \
        --cases bs1:1024,bs1:65536,bs1cp:65536,mtp:1024,dflash:1024,prefill:8192 --rounds 200 [--wide 64]

Speculative modes run a real chunked prefill of ``--ctx`` uniform-random tokens (target and draft
together) and then replay the captured round graph; tokens per round come from the control block, so
``tok/s = committed tokens / time``.  Batch-1 long-context cases are timing fixtures: the committed
length is set to ``--ctx`` over a zero-filled cache (what the reference does for its long-context
timings, ``nex_n2_5_pro/decode_engine.py:687-723``), because attention time depends on the length of
the cache and not on its contents.  ``prefill:N`` times the engine's own prefill of N tokens (8-row steps, or wide
chunks with ``--wide``).  Timing is CUDA events around back-to-back replays after warm-up,
barrier + synchronise on both sides, MAX over ranks; rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="mtp:1024", help="comma list of mode:ctx with mode in bs1, bs1cp, mtp, mtpcp, dflash, dflashcp, prefill; run in order on one engine")
    ap.add_argument("--wide", type=int, default=0, help="rows per wide prefill chunk for the prefills this tool runs (0 = 8-row steps)")
    ap.add_argument("--rounds", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    from ..config import full_config
    from ..decode_engine import DecodeEngine
    from ..models.reference import synthetic_prompt
    from ..runtime.control import Ctl
    from ..serve.process_supervisor import launch_geometry
    from ..utils.bench import tp_max
    from ..weights import random_rank_model

    cases = [(c.split(":")[0], int(c.split(":")[1])) for c in a.cases.split(",") if c]
    want_cp = any(m.endswith("cp") for m, _ in cases)
    rank, world, local = launch_geometry()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    layers = a.layers or (60 if world >= 8 else 4)
    cfg = full_config().truncated(layers) if layers < 60 else full_config()
    cache_len = max(c for _, c in cases) + (a.rounds + a.warmup + 40) * 8 + 1024
    t0 = time.time()
    model = random_rank_model(cfg, world, rank, dev, seed=a.seed, cp=want_cp)
    eng = DecodeEngine(rank, world, dev, cp=want_cp, ext=model, cfg=cfg, max_rows=8, cache_len=cache_len)
    build_s = time.time() - t0
    blocks = {}

    def spec_block(kind):
        if kind in blocks:
            return blocks[kind]
        if kind == "mtp":
            from ..mtp import MtpDraft
            from ..mtp.weights import random_mtp_checkpoint, shard_mtp

            blocks[kind] = MtpDraft(eng, shard_mtp(random_mtp_checkpoint(cfg, seed=a.seed + 7, device=dev), cfg, world, rank, dev, eng.head.w))
        else:
            from dataclasses import replace

            from ..dflash import DFlashBlock, DFlashConfig
            from ..dflash.weights import load_dflash_shard, random_dflash_checkpoint

            dc = DFlashConfig()
            if cfg.n_layers <= max(dc.target_layer_ids):
                step = max(cfg.n_layers // dc.n_taps, 1)
                dc = replace(dc, target_layer_ids=tuple(sorted({min(i * step, cfg.n_layers - 1) for i in range(dc.n_taps)})))
            dc.validate_kernel_contract(cfg, world)
            blocks[kind] = DFlashBlock(eng, dc, load_dflash_shard(random_dflash_checkpoint(dc, seed=a.seed + 11, device=dev), dc, world, rank, dev))
        return blocks[kind]

    worst = 0
    for mode, ctx in cases:
        use_cp = bool(mode.endswith("cp") and eng.cp)
        kind = mode[:-2] if mode.endswith("cp") else mode
        t0 = time.time()
        prompt = synthetic_prompt(cfg.vocab, ctx, seed=1)
        eng.set_forced_commit(0)
        if kind == "prefill":
            # the engine's own prefill of ctx tokens: second call timed (the first captures the step / chunk graphs)
            eng.capture(8)
            eng.prefill(prompt, chunk=8, wide=a.wide)
            torch.cuda.synchronize(dev)
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.prefill(prompt, chunk=8, wide=a.wide)
            e1.record()
            torch.cuda.synchronize(dev)
            ms = tp_max(e0.elapsed_time(e1), dev)
            status = eng.status_max()
            worst = max(worst, status)
            if rank == 0:
                print(json.dumps({"mode": "prefill", "ctx": ctx, "n_gpus": world, "layers": layers, "wide": a.wide, "ms": round(ms, 2),
                                  "tok_s": round(ctx / ms * 1e3, 1), "status": status, "multicast": bool(eng.ctx.channel.multicast),
                                  "build_s": round(build_s, 1)}), flush=True)
            if status:
                break
            continue
        if kind == "bs1":
            eng.reset(first_token=prompt[0], committed_len=ctx)
            graph, mean10 = eng.capture(1, cp=use_cp), 10
        elif kind == "mtp":
            from ..mtp import capture_round

            block = spec_block("mtp")
            block.prefill(prompt, chunk=8, wide=a.wide)
            mean10 = 30
            eng.set_forced_commit(0, seed=1234, mean10=mean10)
            graph = capture_round(block, cp=use_cp)
        else:
            from ..dflash import capture_request

            block = spec_block("dflash")
            block.prefill(prompt, wide=a.wide)
            mean10 = 50
            eng.set_forced_commit(0, seed=1234, mean10=mean10)
            graph = capture_request(block, cp=use_cp)
        setup_s = time.time() - t0
        for _ in range(a.warmup):
            graph.replay()
        torch.cuda.synchronize(dev)
        start_len = int(eng.ctx.ctl[Ctl.COMMITTED_LEN].item())
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.rounds):
            graph.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        ms = tp_max(e0.elapsed_time(e1), dev)
        tokens = int(eng.ctx.ctl[Ctl.COMMITTED_LEN].item()) - start_len
        status = eng.status_max()
        worst = max(worst, status)
        if rank == 0:
            print(json.dumps({
                "mode": kind, "ctx": ctx, "cp": use_cp, "n_gpus": world, "layers": layers, "rounds": a.rounds, "warmup": a.warmup,
                "round_us": round(1e3 * ms / a.rounds, 2), "tokens_per_round": round(tokens / a.rounds, 3), "tok_s": round(tokens / (ms / 1e3), 2),
                "forced_mean_accept": mean10 / 10 if kind != "bs1" else None, "status": status,
                "prefill": "timing fixture (committed length set over a zero cache)" if kind == "bs1" else "engine chunked prefill (8-row steps)",
                "multicast": bool(eng.ctx.channel.multicast), "setup_s": round(setup_s, 1), "build_s": round(build_s, 1),
            }), flush=True)
        if status:
            break
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if worst == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
