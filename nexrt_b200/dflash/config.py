"""DFlash block-draft configuration and the contract between a draft ``config.json`` and the kernels.

Geometry and validation follow the reference's ``DFlashConfig`` / ``validate_kernel_contract``
(``nex_n2_5_pro/dflash/config.py:30-46,50-148``): a 6-layer dense BF16 stack (5 sliding-window
layers of 4096 + 1 full-attention layer), hidden 4096, 32 query / 8 kv heads of 128, MLP 12288,
``fc [4096, 8 * 4096]`` over 8 target tap layers, block size 8.  Environment knobs keep the reference
names: ``NEXRT_DFLASH_DIR``, ``NEXRT_DFLASH_CONFIG``, ``NEXRT_DFLASH_WEIGHTS`` (config.py:26-28).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Tuple

from ..config import ModelConfig

DFLASH_DIR = Path(os.environ.get("NEXRT_DFLASH_DIR", "/path/to/dflash"))
DFLASH_CONFIG = Path(os.environ.get("NEXRT_DFLASH_CONFIG", str(DFLASH_DIR / "config.json")))
DFLASH_WEIGHTS = Path(os.environ.get("NEXRT_DFLASH_WEIGHTS", str(DFLASH_DIR / "model.safetensors")))


@dataclass(frozen=True)
class DFlashConfig:
    hidden: int = 4096
    n_layers: int = 6
    n_q_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    mlp_inter: int = 12288
    sliding_window: int = 4096
    layer_types: Tuple[str, ...] = ("sliding",) * 5 + ("full",)
    target_layer_ids: Tuple[int, ...] = (1, 9, 17, 25, 33, 41, 49, 57)
    block_size: int = 8
    mask_token_id: int = 248319
    rope_theta: float = 1.0e7
    rotary_dim: int = 128
    rms_eps: float = 1e-6
    vocab: int = 248320

    @property
    def n_taps(self) -> int:
        return len(self.target_layer_ids)

    def validate_kernel_contract(self, target: ModelConfig, tp: int = 1) -> None:
        """Raise ``ValueError`` unless the kernels can run this draft next to ``target``."""
        problems = []
        if self.hidden != target.hidden:
            problems.append(f"draft hidden {self.hidden} != target hidden {target.hidden}")
        if self.vocab != target.vocab:
            problems.append("the draft shares the target's embedding and LM head: vocab must match")
        if self.block_size != 8:
            problems.append("the verify step carries exactly 8 rows")
        if self.head_dim not in (128, 256):
            problems.append("attention kernels are instantiated for head_dim 128 and 256")
        if len(self.layer_types) != self.n_layers or any(t not in ("sliding", "full") for t in self.layer_types):
            problems.append("layer_types must name n_layers entries of 'sliding' or 'full'")
        if any(not 0 <= l < target.n_layers for l in self.target_layer_ids):
            problems.append("target_layer_ids outside the target stack")
        if list(self.target_layer_ids) != sorted(set(self.target_layer_ids)):
            problems.append("target_layer_ids must be strictly increasing")
        if self.n_q_heads % tp or (self.n_kv_heads % tp and tp % self.n_kv_heads):
            problems.append(f"heads not divisible by tp={tp}")
        if self.mlp_inter % (32 * tp) or (self.n_taps * self.hidden) % (32 * tp):
            problems.append(f"MLP / fc widths not divisible by 32*tp={32 * tp}")
        if self.hidden > 4096:
            problems.append("norm prologue supports hidden <= 4096")
        if not 0 <= self.mask_token_id < self.vocab:
            problems.append("mask_token_id outside the vocabulary")
        if self.rotary_dim > self.head_dim or self.rotary_dim % 2:
            problems.append("rotary_dim must be even and at most head_dim")
        if problems:
            raise ValueError("DFlash draft does not match the kernel contract: " + "; ".join(problems))

    @classmethod
    def from_json(cls, path=None) -> "DFlashConfig":
        cfg = json.loads(Path(path or DFLASH_CONFIG).read_text())
        d = cfg.get("dflash_config", {})
        types = tuple("sliding" if t in ("sliding", "sliding_attention") else "full" for t in cfg.get("layer_types", cls.layer_types))
        return cls(
            hidden=cfg.get("hidden_size", cls.hidden), n_layers=cfg.get("num_hidden_layers", cls.n_layers),
            n_q_heads=cfg.get("num_attention_heads", cls.n_q_heads), n_kv_heads=cfg.get("num_key_value_heads", cls.n_kv_heads),
            head_dim=cfg.get("head_dim", cls.head_dim), mlp_inter=cfg.get("intermediate_size", cls.mlp_inter),
            sliding_window=cfg.get("sliding_window", cls.sliding_window), layer_types=types,
            target_layer_ids=tuple(d.get("target_layer_ids", cfg.get("target_layer_ids", cls.target_layer_ids))),
            block_size=cfg.get("block_size", d.get("block_size", cls.block_size)),
            mask_token_id=d.get("mask_token_id", cfg.get("mask_token_id", cls.mask_token_id)),
            rope_theta=cfg.get("rope_theta", cls.rope_theta), rms_eps=cfg.get("rms_norm_eps", cls.rms_eps),
            vocab=cfg.get("vocab_size", cls.vocab), rotary_dim=cfg.get("rotary_dim", cfg.get("head_dim", cls.head_dim)),
        )


def shrunk_dflash_config(target: ModelConfig) -> DFlashConfig:
    """Small draft used with the shrunk target in tests."""
    return DFlashConfig(
        hidden=target.hidden, n_layers=2, n_q_heads=8, n_kv_heads=2, head_dim=128, mlp_inter=512, sliding_window=16,
        layer_types=("sliding", "full"), target_layer_ids=tuple(range(min(2, target.n_layers))), block_size=8,
        mask_token_id=target.vocab - 1, rope_theta=target.rope_theta, rotary_dim=128, vocab=target.vocab,
    )
