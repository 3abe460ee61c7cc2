"""Offline prefill-state extractor: run the engine's own chunked prefill on a prompt and save what a
later decode run needs to start at that boundary.

Per rank ``prefill_state_rank<r>.pt`` = ``{rank, tp, L, prompt_ids, first_token, layers{idx: {kind,
k_cache, v_cache | conv_state, recurrent_state}}}`` and, from rank 0, ``prefill_meta.pt`` and
``golden.pt`` (the greedy continuation used as a teacher-forced comparison stream).  Same file set as
the reference's ``sglang_prefill/extract_state.py:248-281``, where the states come out of SGLang's
pools; here they are the engine's own caches, so no re-rotation of K is needed.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 -m nexrt_b200.extract_state \
        --length 1024 --out /data/nexrt-state/prefill_state_60_1024
"""

from __future__ import annotations

import argparse
import os
from pathlib import Path
from typing import Dict, List, Sequence

import torch


def state_dir(root, n_layers: int, length: int) -> Path:
    return Path(root) / f"prefill_state_{n_layers}_{length}"


def save_state(engine, prompt_ids: Sequence[int], out_dir, golden: Sequence[int] = ()) -> Path:
    """Write this rank's state file (and the meta / golden files from rank 0)."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    state = engine.export_state()
    state["prompt_ids"] = [int(t) for t in prompt_ids]
    state["layers"] = {k: {n: (v.cpu() if torch.is_tensor(v) else v) for n, v in d.items()} for k, d in state["layers"].items()}
    path = out / f"prefill_state_rank{engine.rank}.pt"
    tmp = path.with_suffix(f".{os.getpid()}.tmp")
    torch.save(state, tmp)
    os.replace(tmp, path)
    if engine.rank == 0:
        torch.save({"tp": engine.world, "L": state["L"], "n_layers": engine.cfg.n_layers, "first_token": state["first_token"],
                    "prompt_ids": state["prompt_ids"]}, out / "prefill_meta.pt")
        if golden:
            torch.save({"tokens": [int(t) for t in golden]}, out / "golden.pt")
    return path


def load_state(engine, in_dir) -> Dict:
    """Install ``prefill_state_rank<r>.pt`` of this rank; returns the loaded dict."""
    state = torch.load(Path(in_dir) / f"prefill_state_rank{engine.rank}.pt", map_location="cpu", weights_only=False)
    if int(state["tp"]) != engine.world:
        raise ValueError(f"state was written at tp={state['tp']}, engine runs tp={engine.world}")
    engine.load_prefill(state)
    return state


def make_prompt(length: int, vocab: int, tokenizer_dir=None, seed: int = 1) -> List[int]:
    if tokenizer_dir:
        from transformers import AutoTokenizer

        from .real_prompts import build_real_prompt

        return build_real_prompt(length, AutoTokenizer.from_pretrained(tokenizer_dir))
    from .models.reference import synthetic_prompt

    return synthetic_prompt(vocab, length, seed=seed)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--length", type=int, required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--layers", type=int, default=int(os.environ.get("NEXRT_NLAYERS", "60")))
    ap.add_argument("--layers-dir", default=None)
    ap.add_argument("--tokenizer", default=os.environ.get("NEXRT_MODEL_DIR"))
    ap.add_argument("--golden", type=int, default=32, help="greedy continuation tokens to record")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    import torch.distributed as dist

    from .config import full_config
    from .decode_engine import DecodeEngine
    from .sampling import GREEDY
    from .serve.process_supervisor import launch_geometry
    from .weights import load_rank_model, random_rank_model

    rank, world, local = launch_geometry()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = full_config().truncated(a.layers)
    model = (load_rank_model(cfg, a.layers_dir, world, rank, dev) if a.layers_dir
             else random_rank_model(cfg, world, rank, dev, seed=a.seed))
    eng = DecodeEngine(rank, world, dev, cp=False, ext=model, cfg=cfg, max_rows=8, cache_len=a.length + a.golden + 64)
    eng.head.set_sampling_config(0, *GREEDY)
    prompt = make_prompt(a.length, cfg.vocab, a.tokenizer)
    first = eng.prefill(prompt)
    snap = eng._snapshot()
    golden = [first] + eng.generate(max_new=a.golden - 1) if a.golden > 1 else [first]
    eng._restore(snap)
    path = save_state(eng, prompt, a.out, golden)
    if rank == 0:
        print(f"@@ STATE L={a.length} first_token={first} golden={len(golden)} -> {path.parent}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
