"""DFlash draft weights: random initialisation, checkpoint names and rank-local BF16 shards.

Counterpart of ``nex_n2_5_pro/dflash/weights.py:94-340`` (rank-local shard loader and fragment
prepacks).  No prepack is needed here: the tensor-core projection kernel consumes plain row-major
BF16 rows, so a shard is a row / column slice of the checkpoint tensor:

* ``wqkv [(q_local + 2 kv_local) * hd, H]`` (q heads, then k heads, then v heads of this rank),
* ``wo [H, q_local * hd]``, ``wgu [2 * I_local, H]`` (gate rows then up rows), ``wdown [H, I_local]``,
* ``fc [H, n_taps * H / tp]``: this rank's window of the concatenated target features.
"""

from __future__ import annotations

from typing import Dict

import torch

from .config import DFlashConfig

STD = 0.02


def random_dflash_checkpoint(dc: DFlashConfig, seed: int = 11, device="cpu") -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device=device).manual_seed(seed)
    bf = torch.bfloat16
    rn = lambda *shape: (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * STD).to(bf)
    H, hd = dc.hidden, dc.head_dim
    out = {"fc.weight": rn(H, dc.n_taps * H), "hidden_norm.weight": rn(H), "norm.weight": rn(H)}
    for l in range(dc.n_layers):
        p = f"layers.{l}."
        out[p + "input_layernorm.weight"] = rn(H)
        out[p + "post_attention_layernorm.weight"] = rn(H)
        out[p + "self_attn.q_proj.weight"] = rn(dc.n_q_heads * hd, H)
        out[p + "self_attn.k_proj.weight"] = rn(dc.n_kv_heads * hd, H)
        out[p + "self_attn.v_proj.weight"] = rn(dc.n_kv_heads * hd, H)
        out[p + "self_attn.o_proj.weight"] = rn(H, dc.n_q_heads * hd)
        out[p + "self_attn.q_norm.weight"] = rn(hd)
        out[p + "self_attn.k_norm.weight"] = rn(hd)
        out[p + "mlp.gate_proj.weight"] = rn(dc.mlp_inter, H)
        out[p + "mlp.up_proj.weight"] = rn(dc.mlp_inter, H)
        out[p + "mlp.down_proj.weight"] = rn(H, dc.mlp_inter)
    return out


def load_dflash_shard(ckpt: Dict[str, torch.Tensor], dc: DFlashConfig, tp: int, rank: int, device) -> Dict:
    """Rank-local BF16 shard in kernel layout (reference ``load_dflash_shard``, weights.py:94-190)."""
    hd, H = dc.head_dim, dc.hidden
    q_local = dc.n_q_heads // tp
    if tp <= dc.n_kv_heads:
        kv_local, kv0 = dc.n_kv_heads // tp, rank * (dc.n_kv_heads // tp)
    else:
        kv_local, kv0 = 1, rank // (tp // dc.n_kv_heads)
    I_local = dc.mlp_inter // tp
    win = dc.n_taps * H // tp
    g1 = lambda t: (1.0 + t.float()).contiguous().to(device)
    d = lambda t: t.to(torch.bfloat16).contiguous().to(device)
    layers = []
    for l in range(dc.n_layers):
        p = f"layers.{l}."
        q = ckpt[p + "self_attn.q_proj.weight"][rank * q_local * hd : (rank + 1) * q_local * hd]
        k = ckpt[p + "self_attn.k_proj.weight"][kv0 * hd : (kv0 + kv_local) * hd]
        v = ckpt[p + "self_attn.v_proj.weight"][kv0 * hd : (kv0 + kv_local) * hd]
        gate = ckpt[p + "mlp.gate_proj.weight"][rank * I_local : (rank + 1) * I_local]
        up = ckpt[p + "mlp.up_proj.weight"][rank * I_local : (rank + 1) * I_local]
        layers.append({
            "in_ln": g1(ckpt[p + "input_layernorm.weight"]), "post_ln": g1(ckpt[p + "post_attention_layernorm.weight"]),
            "wqkv": d(torch.cat([q, k, v], 0)), "wkv": d(torch.cat([k, v], 0)),
            "wo": d(ckpt[p + "self_attn.o_proj.weight"][:, rank * q_local * hd : (rank + 1) * q_local * hd]),
            "qn": g1(ckpt[p + "self_attn.q_norm.weight"]), "kn": g1(ckpt[p + "self_attn.k_norm.weight"]),
            "wgu": d(torch.cat([gate, up], 0)),
            "wdown": d(ckpt[p + "mlp.down_proj.weight"][:, rank * I_local : (rank + 1) * I_local]),
            "window": dc.sliding_window if dc.layer_types[l] == "sliding" else 0,
        })
    return {
        "layers": layers, "q_local": q_local, "kv_local": kv_local, "I_local": I_local, "win": win, "win0": rank * win,
        "fc": d(ckpt["fc.weight"][:, rank * win : (rank + 1) * win]),
        "hidden_ln": g1(ckpt["hidden_norm.weight"]), "final_ln": g1(ckpt["norm.weight"]),
    }


def expected_shapes(dc: DFlashConfig) -> Dict[str, tuple]:
    """Every tensor of a DFlash draft checkpoint with the shape the kernels' geometry requires."""
    H, hd = dc.hidden, dc.head_dim
    out = {"fc.weight": (H, dc.n_taps * H), "hidden_norm.weight": (H,), "norm.weight": (H,)}
    for l in range(dc.n_layers):
        p = f"layers.{l}."
        out.update({
            p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
            p + "self_attn.q_proj.weight": (dc.n_q_heads * hd, H), p + "self_attn.k_proj.weight": (dc.n_kv_heads * hd, H),
            p + "self_attn.v_proj.weight": (dc.n_kv_heads * hd, H), p + "self_attn.o_proj.weight": (H, dc.n_q_heads * hd),
            p + "self_attn.q_norm.weight": (hd,), p + "self_attn.k_norm.weight": (hd,),
            p + "mlp.gate_proj.weight": (dc.mlp_inter, H), p + "mlp.up_proj.weight": (dc.mlp_inter, H),
            p + "mlp.down_proj.weight": (H, dc.mlp_inter),
        })
    return out


def check_dflash_checkpoint(ckpt, dc: DFlashConfig) -> None:
    """The draft geometry is fixed: a checkpoint with a missing tensor or another shape is refused before anything is
    copied (reference ``_require_shape`` at boot, dflash/weights.py:117-142).  ``ckpt`` is a dict of tensors or a
    ``weights.TensorFiles`` mapping, whose shapes come from the file header."""
    shape_of = ckpt.shape if hasattr(ckpt, "shape") and callable(ckpt.shape) else (lambda k: tuple(ckpt[k].shape))
    problems = []
    for key, want in expected_shapes(dc).items():
        if key not in ckpt:
            problems.append(f"{key}: missing")
        elif tuple(shape_of(key)) != want:
            problems.append(f"{key}: shape {tuple(shape_of(key))}, expected {want}")
    if problems:
        more = f" (+{len(problems) - 6} more)" if len(problems) > 6 else ""
        raise ValueError("DFlash checkpoint does not match the draft geometry: " + "; ".join(problems[:6]) + more)


def load_dflash_files(dc: DFlashConfig, tp: int, rank: int, device, weights_path=None) -> Dict:
    """This rank's shard straight from the draft's ``model.safetensors`` (default: ``NEXRT_DFLASH_WEIGHTS`` /
    ``NEXRT_DFLASH_DIR``), one tensor on the host at a time, after the geometry check."""
    from ..weights import TensorFiles
    from .config import DFLASH_WEIGHTS

    files = TensorFiles([weights_path or DFLASH_WEIGHTS], prefault=False)
    try:
        check_dflash_checkpoint(files, dc)
        return load_dflash_shard(files, dc, tp, rank, device)
    finally:
        files.close()
