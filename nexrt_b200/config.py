"""Model geometry and tensor-parallel shard geometry.

The geometry constants of the served model (Nex-N2.5-Pro) mirror the reference's
``nex_n2_5_pro/config.py:32-46`` (hidden 4096, 60 layers, full attention on every 4th layer,
vocab 248320, eps 1e-6), ``nex_n2_5_pro/attn.py:63-78`` (32 q / 2 kv heads of 256, rotary 64,
theta 1e7), ``nex_n2_5_pro/gdn.py:53`` (16 qk / 64 v heads of 128, conv width 4) and
``nex_n2_5_pro/moe.py:52`` (512 experts, top-10, intermediate 1024, one shared expert).

Unlike the reference, whose shard functions raise unless ``tp == 8``
(``nex_n2_5_pro/weights.py:85-86``), every shard size here is a function of ``tp`` so the
same engine runs at tensor-parallel 1, 2, 4 and 8, and a shrunk geometry is available for
CPU-only oracle tests.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import Tuple

BLOCK = 128  # edge of one FP8 scale block (128 x 128 weights share one fp32 scale)


def _default_layer_types(n_layers: int, interval: int) -> Tuple[str, ...]:
    return tuple("full" if (layer + 1) % interval == 0 else "linear" for layer in range(n_layers))


@dataclass(frozen=True)
class ModelConfig:
    """Geometry of one hybrid GDN / gated-attention MoE stack."""

    name: str = "nex-n2.5-pro"
    hidden: int = 4096
    vocab: int = 248320
    n_layers: int = 60
    full_attn_interval: int = 4
    layer_types: Tuple[str, ...] = ()
    rms_eps: float = 1e-6
    # gated full attention
    n_q_heads: int = 32
    n_kv_heads: int = 2
    head_dim: int = 256
    rotary_dim: int = 64
    rope_theta: float = 1.0e7
    # gated delta net
    gdn_qk_heads: int = 16
    gdn_v_heads: int = 64
    gdn_dim: int = 128
    conv_kernel: int = 4
    # mixture of experts
    n_experts: int = 512
    top_k: int = 10
    moe_inter: int = 1024
    shared_inter: int = 1024
    # caches
    max_context: int = 256 * 1024
    decode_headroom: int = 1024
    # speculative-decoding state rings (position indexed; the no-alias law is checked by runtime/control.py: ring_no_alias)
    conv_ring: int = 16
    state_ring: int = 9

    def __post_init__(self):
        if not self.layer_types:
            object.__setattr__(
                self, "layer_types", _default_layer_types(self.n_layers, self.full_attn_interval)
            )
        if len(self.layer_types) != self.n_layers:
            raise ValueError("layer_types must have n_layers entries")
        if self.shared_inter != self.moe_inter:
            raise ValueError("the shared expert is stored as expert index n_experts: same width")
        if self.gdn_dim != 128:
            raise ValueError("gated-delta-net kernels are written for head dim 128")
        if self.head_dim not in (128, 256):
            raise ValueError("attention kernels are instantiated for head_dim 128 and 256")

    # ---- derived sizes -------------------------------------------------------------------
    @property
    def cache_len(self) -> int:
        return self.max_context + self.decode_headroom

    @property
    def gdn_key_dim(self) -> int:
        return self.gdn_qk_heads * self.gdn_dim

    @property
    def gdn_value_dim(self) -> int:
        return self.gdn_v_heads * self.gdn_dim

    @property
    def n_linear(self) -> int:
        return sum(1 for t in self.layer_types if t == "linear")

    @property
    def n_full(self) -> int:
        return sum(1 for t in self.layer_types if t == "full")

    def truncated(self, n_layers: int) -> "ModelConfig":
        """Prefix of the stack (the reference's ``NEXRT_NLAYERS`` knob, config.py:42-46)."""
        if not 1 <= n_layers <= self.n_layers:
            raise ValueError(f"n_layers must be in [1, {self.n_layers}], got {n_layers}")
        return replace(self, n_layers=n_layers, layer_types=self.layer_types[:n_layers])

    def max_tp(self) -> int:
        tp = 1
        while tp < 8 and self.supports_tp(tp * 2):
            tp *= 2
        return tp

    def supports_tp(self, tp: int) -> bool:
        try:
            ShardSpec(self, tp, 0)
        except ValueError:
            return False
        return True


def full_config() -> ModelConfig:
    return ModelConfig()


def shrunk_config() -> ModelConfig:
    """The CPU-oracle geometry: hidden 1024, vocab 4096, one GDN layer and one attention layer,
    16 experts top-4 of width 256 plus one shared expert."""
    return ModelConfig(
        name="nex-shrunk",
        hidden=1024,
        vocab=4096,
        n_layers=2,
        layer_types=("linear", "full"),
        n_q_heads=8,
        n_kv_heads=2,
        head_dim=128,
        rotary_dim=32,
        gdn_qk_heads=4,
        gdn_v_heads=4,
        gdn_dim=128,
        n_experts=16,
        top_k=4,
        moe_inter=256,
        shared_inter=256,
        max_context=4096,
        decode_headroom=256,
    )


def rank_shard_config() -> ModelConfig:
    """A two-layer model whose GLOBAL shapes are one rank's shard of the full geometry at tensor-parallel 8: hidden 4096,
    4 query heads over 1 kv head of dim 256, 2 + 8 gated-delta-net heads, 512 experts top-10 of width 128, 31 040
    vocabulary rows.  Run at tp = 1 it drives exactly the kernel instantiations of the 8-GPU deployment (head_dim-256
    attention, 528-row router with top-10, K = 4096 fronts, the 31 040-row head) while staying small enough for the
    fp32 oracle, which keeps the experts in FP8 and dequantises the handful a token selects."""
    return ModelConfig(
        name="nex-rank-shard",
        hidden=4096,
        vocab=31040,
        n_layers=2,
        layer_types=("linear", "full"),
        n_q_heads=4,
        n_kv_heads=1,
        head_dim=256,
        rotary_dim=64,
        gdn_qk_heads=2,
        gdn_v_heads=8,
        gdn_dim=128,
        n_experts=512,
        top_k=10,
        moe_inter=128,
        shared_inter=128,
        max_context=2048,
        decode_headroom=256,
    )


def shrunk_tp8_config() -> ModelConfig:
    """Shrunk geometry that splits 8 ways (every head count a multiple of 8, expert width 8 x 128): the numerics of the
    8-rank deployment against the CPU oracle.  2 kv heads over 8 ranks also gives context-parallel groups of 4, the
    reference's deployment geometry (``nex_n2_5_pro/attn_cp.py:76-174``)."""
    return replace(shrunk_config(), name="nex-shrunk-tp8", n_q_heads=8, gdn_qk_heads=8, gdn_v_heads=8, moe_inter=1024, shared_inter=1024)


def shrunk_cp_config() -> ModelConfig:
    """Shrunk geometry that can be split 4 ways: 2 kv heads over 4 ranks gives context-parallel groups
    of 2 (multi-GPU tests of the CP arm)."""
    return replace(shrunk_config(), name="nex-shrunk-cp", moe_inter=512, shared_inter=512)


@dataclass(frozen=True)
class ShardSpec:
    """What one tensor-parallel rank owns.

    Attention is head parallel with the kv head replicated inside the group of ranks that
    share it (reference ``weights.py:84-105``: ``kv_head = rank // (tp / n_kv)``); the gated
    delta net is head parallel; every expert is split along its intermediate dimension
    (reference ``moe.py:145-171``); the LM head is vocab parallel (``head.py:19-25``).
    """

    cfg: ModelConfig
    tp: int
    rank: int
    q_heads: int = field(init=False)
    kv_heads: int = field(init=False)
    kv_head0: int = field(init=False)
    cp_size: int = field(init=False)
    cp_rank: int = field(init=False)
    gdn_qk: int = field(init=False)
    gdn_v: int = field(init=False)
    inter: int = field(init=False)
    vocab: int = field(init=False)

    def __post_init__(self):
        c, tp, rank = self.cfg, self.tp, self.rank
        if tp not in (1, 2, 4, 8) or not 0 <= rank < tp:
            raise ValueError(f"bad tensor-parallel geometry tp={tp} rank={rank}")
        if c.n_q_heads % tp or c.gdn_qk_heads % tp or c.gdn_v_heads % tp or c.vocab % tp:
            raise ValueError(f"{c.name}: heads/vocab not divisible by tp={tp}")
        if c.moe_inter % tp or (c.moe_inter // tp) % BLOCK:
            raise ValueError(f"{c.name}: expert width {c.moe_inter} cannot be split {tp} ways")
        s = object.__setattr__
        s(self, "q_heads", c.n_q_heads // tp)
        if tp <= c.n_kv_heads:
            s(self, "kv_heads", c.n_kv_heads // tp)
            s(self, "kv_head0", rank * (c.n_kv_heads // tp))
            s(self, "cp_size", 1)
            s(self, "cp_rank", 0)
        else:
            group = tp // c.n_kv_heads
            s(self, "kv_heads", 1)
            s(self, "kv_head0", rank // group)
            s(self, "cp_size", group)
            s(self, "cp_rank", rank % group)
        s(self, "gdn_qk", c.gdn_qk_heads // tp)
        s(self, "gdn_v", c.gdn_v_heads // tp)
        s(self, "inter", c.moe_inter // tp)
        s(self, "vocab", c.vocab // tp)

    # row counts of the fused projections of one rank
    @property
    def gdn_qkv_rows(self) -> int:
        return (2 * self.gdn_qk + self.gdn_v) * self.cfg.gdn_dim

    @property
    def gdn_front_rows(self) -> int:
        return self.gdn_qkv_rows + self.gdn_v * self.cfg.gdn_dim

    @property
    def gdn_local(self) -> int:
        return self.gdn_v * self.cfg.gdn_dim

    @property
    def attn_front_rows(self) -> int:
        return (2 * self.q_heads + 2 * self.kv_heads) * self.cfg.head_dim

    @property
    def attn_local(self) -> int:
        return self.q_heads * self.cfg.head_dim

    @property
    def cp_group(self) -> Tuple[int, ...]:
        base = (self.rank // self.cp_size) * self.cp_size
        return tuple(range(base, base + self.cp_size))


# ---- environment knobs (same names as the reference, config.py:29,42 / decode_engine.py:69-71)
LAYERS_DIR = Path(os.environ.get("NEXRT_LAYERS_DIR", "/path/to/nexrt-layers"))
STATE_DIR = Path(os.environ.get("NEXRT_STATE_DIR", "/path/to/nexrt-state"))


def active_config() -> ModelConfig:
    """Full geometry truncated by ``NEXRT_NLAYERS`` (1..60)."""
    cfg = full_config()
    n = int(os.environ.get("NEXRT_NLAYERS", str(cfg.n_layers)))
    return cfg.truncated(n) if n != cfg.n_layers else cfg
