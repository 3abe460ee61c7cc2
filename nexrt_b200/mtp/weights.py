"""MTP draft-layer weights: random initialisation, checkpoint names, tensor-parallel shards.

Names follow the reference loader (``nex_n2_5_pro/mtp/weights.py:52-79,135-174``): ``mtp.fc.weight``
``[H, 2H]`` bf16, ``mtp.pre_fc_norm_embedding.weight``, ``mtp.pre_fc_norm_hidden.weight``,
``mtp.norm.weight`` and one decoder layer ``mtp.layers.0.*`` with the target's attention / MoE
geometry; the embedding and the LM head are the target's.  ``mtp.fc`` is quantised to FP8 with
128x128 block scales at load (the reference does the same) and column-sliced over the ranks:
rank r multiplies its window of ``cat[norm_e(emb) | norm_h(hidden)]`` and the partial products are
all-reduced by the fused out-projection kernel.
"""

from __future__ import annotations

from dataclasses import replace
from typing import Dict

import torch

from ..config import ModelConfig, ShardSpec
from ..quant import FP8, quantize_blockwise
from ..weights import INIT_STD, PFX, _gamma, random_layer, shard_attention, shard_moe

MTP_BASE = "mtp.layers.0."


def random_mtp_checkpoint(cfg: ModelConfig, seed: int = 7, device="cpu") -> Dict[str, torch.Tensor]:
    """Random-init MTP tensors under checkpoint names (target geometry, FP8 block scales)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    H, bf = cfg.hidden, torch.bfloat16
    rn = lambda *shape: torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * INIT_STD
    # one full-attention layer of the target's geometry
    one = replace(cfg, n_layers=1, layer_types=("full",))
    layer = random_layer(one, 0, gen, device)
    out = {k.replace(f"{PFX}layers.0.", MTP_BASE): v for k, v in layer.items()}
    out["mtp.fc.weight"] = rn(H, 2 * H).to(bf)
    out["mtp.pre_fc_norm_embedding.weight"] = rn(H).to(bf)
    out["mtp.pre_fc_norm_hidden.weight"] = rn(H).to(bf)
    out["mtp.norm.weight"] = rn(H).to(bf)
    return out


def shard_mtp(ckpt: Dict[str, torch.Tensor], cfg: ModelConfig, tp: int, rank: int, device, target_head: Dict) -> Dict:
    """Kernel-layout MTP tensors of one rank.  ``target_head`` is the target's ``head`` dict (shared
    embedding, LM head shard and final norm): the draft owns no copy of them, so they must still be resident
    (reference mtp/weights.py: the draft reuses the target's head and refuses a released one)."""
    missing = [k for k in ("embed", "lm_head", "final_ln") if not isinstance((target_head or {}).get(k), torch.Tensor)]
    if missing:
        raise ValueError(f"the MTP draft shares the target's head tensors, which are not resident: {missing}")
    spec = ShardSpec(cfg, tp, rank)
    H = cfg.hidden
    win = 2 * H // tp
    fq, fs = quantize_blockwise(ckpt["mtp.fc.weight"].float())
    d = lambda t: t.contiguous().to(device)
    return {
        "fc_w": d(fq.view(torch.uint8)[:, rank * win : (rank + 1) * win]).view(FP8),
        "fc_s": d(fs[:, rank * win // 128 : (rank + 1) * win // 128]),
        "win0": rank * win,
        "win": win,
        "ge": d(_gamma(ckpt["mtp.pre_fc_norm_embedding.weight"])),
        "gh": d(_gamma(ckpt["mtp.pre_fc_norm_hidden.weight"])),
        "gf": target_head["final_ln"],
        "mixer": shard_attention(ckpt, cfg, 0, spec, device, base=MTP_BASE),
        "moe": shard_moe(ckpt, cfg, 0, spec, device, base=MTP_BASE),
        "head": {"final_ln": d(_gamma(ckpt["mtp.norm.weight"])), "lm_head": target_head["lm_head"], "embed": target_head["embed"]},
    }


def load_mtp_files(cfg: ModelConfig, layers_dir, tp: int, rank: int, device, target_head: Dict) -> Dict:
    """This rank's MTP tensors straight from ``mtp.safetensors`` of a layer directory, one tensor on the host at a time.
    Nothing of the target is read again: the embedding, the LM head shard and the final norm are the resident ones."""
    from pathlib import Path

    from ..weights import TensorFiles

    path = Path(layers_dir) / "mtp.safetensors"
    if not path.is_file():
        raise FileNotFoundError(f"{path}: the layer directory holds no MTP weights")
    files = TensorFiles([path], prefault=False)
    try:
        return shard_mtp(files, cfg, tp, rank, device, target_head)
    finally:
        files.close()
