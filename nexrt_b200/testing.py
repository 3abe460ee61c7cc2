"""Small fixtures shared by the tests, the smoke entry point and the examples: a shrunk random
model, its CPU oracle and an engine over it."""

from __future__ import annotations

import functools

import torch

from .config import ModelConfig, shrunk_config, shrunk_cp_config
from .weights import random_checkpoint, shard_model


@functools.lru_cache(maxsize=4)
def shrunk_checkpoint(seed: int = 0, cp: bool = False):
    cfg = shrunk_cp_config() if cp else shrunk_config()
    return cfg, random_checkpoint(cfg, seed)


def make_engine(cfg: ModelConfig, ckpt, rank=0, world=1, device=None, group=None, max_rows=8, cache_len=None, cp=False, budget_ms=None):
    from .decode_engine import DecodeEngine

    device = device or torch.device("cuda", torch.cuda.current_device())
    model = shard_model(ckpt, cfg, world, rank, device, cp=cp)
    return DecodeEngine(rank, world, device, cp=cp, ext=model, cfg=cfg, group=group, max_rows=max_rows,
                        cache_len=cache_len or cfg.cache_len, budget_ms=budget_ms)


def gather_logits(engine, rows: int) -> torch.Tensor:
    """fp32 logits ``[rows, vocab_local]`` of the last step (engine.head.enable_logits() first)."""
    torch.cuda.synchronize()
    return engine.head.logits[:rows].float().cpu()
