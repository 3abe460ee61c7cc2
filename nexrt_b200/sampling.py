"""Sampling parameters and the fixed 64-byte device buffer they travel in.

Same contract as the reference (``nex_n2_5_pro/sampling.py:30-81``): ``uint64[8]`` =
``[seed, (f32 temperature | f32 top_p), top_k, 5 reserved]``, ``top_k <= 28``, defaults
``(0.6, 0.95, 20)`` overridable by a ``generation_config.json`` next to the weights.  Parameters
live in device memory so a captured graph never needs recapture when a request changes them.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Any, List, Mapping, Optional, Tuple

import numpy as np

MAX_TOP_K = 28
SAMPLING_WORDS = 8
DEFAULT_SAMPLING = (0.6, 0.95, 20)
GREEDY = (0.0, 1.0, 1)


def _as_f32(name: str, value: Any) -> np.float32:
    """``value`` rounded the way the device will hold it; anything float32 cannot represent is refused."""
    try:
        wide = float(value)
    except (TypeError, ValueError) as error:
        raise ValueError(f"{name} must be a real number") from error
    if wide != wide or wide in (float("inf"), float("-inf")):
        raise ValueError(f"{name} must be finite")
    with np.errstate(over="ignore"):
        narrow = np.float32(wide)
    if not np.isfinite(narrow):
        raise ValueError(f"{name} must fit float32")
    if wide != 0.0 and narrow == 0.0:
        raise ValueError(f"{name} must not underflow float32")
    return narrow


@dataclass(frozen=True)
class SamplingConfig:
    """One request's sampling parameters, already in device precision.  ``pack(seed)`` gives the eight 64-bit words
    of the device buffer: word 0 the seed, word 1 the two float32 bit patterns (temperature low, top_p high), word 2
    top_k, words 3..7 reserved as zero."""

    temperature: float
    top_p: float
    top_k: int

    @classmethod
    def make(cls, temperature: Any, top_p: Any, top_k: Any) -> "SamplingConfig":
        t = _as_f32("temperature", temperature)
        if t < 0:
            raise ValueError("temperature must be >= 0")
        p = _as_f32("top_p", top_p)
        if not (0 < p <= 1):
            raise ValueError("top_p must lie in (0, 1]")
        # an integer type only: True, 2.5 or "3" are not top-k values
        if isinstance(top_k, (bool, np.bool_)) or not isinstance(top_k, (int, np.integer)):
            raise ValueError(f"top_k must be an integer in [1, {MAX_TOP_K}]")
        k = int(top_k)
        if k < 1 or k > MAX_TOP_K:
            raise ValueError(f"top_k must be an integer in [1, {MAX_TOP_K}]")
        return cls(float(t), float(p), k)

    def with_overrides(self, temperature: Any = None, top_p: Any = None, top_k: Any = None) -> "SamplingConfig":
        return SamplingConfig.make(self.temperature if temperature is None else temperature, self.top_p if top_p is None else top_p,
                                   self.top_k if top_k is None else top_k)

    def as_tuple(self) -> Tuple[float, float, int]:
        return (self.temperature, self.top_p, self.top_k)

    def pack(self, seed: int) -> List[int]:
        floats = np.array([self.temperature, self.top_p], dtype="<f4")
        words = np.zeros(SAMPLING_WORDS, dtype=np.uint64)
        words[0] = int(seed) % (1 << 64)
        words[1] = int(floats.view("<u8")[0])
        words[2] = self.top_k
        return [int(w) for w in words.view(np.int64)]      # the buffer is a torch int64 tensor: two's-complement view


def checked_sampling_config(temperature, top_p, top_k) -> Tuple[float, float, int]:
    """Validate and return ``(temperature, top_p, top_k)`` exactly as the device will see them (float32 rounded)."""
    return SamplingConfig.make(temperature, top_p, top_k).as_tuple()


def resolve_sampling_config(defaults, temperature=None, top_p=None, top_k=None) -> Tuple[float, float, int]:
    """Request values over server defaults; ``None`` keeps the default."""
    return SamplingConfig.make(*defaults).with_overrides(temperature, top_p, top_k).as_tuple()


def _generation_config(directory: Optional[str]) -> Mapping[str, Any]:
    if not directory:
        return {}
    path = Path(directory) / "generation_config.json"
    return json.loads(path.read_text()) if path.is_file() else {}


def sampling_defaults(model_dir: Optional[str] = None) -> Tuple[float, float, int]:
    """Server defaults: ``DEFAULT_SAMPLING`` overridden by the checkpoint's ``generation_config.json`` (looked up in
    ``model_dir``, else under ``NEXRT_MODEL_DIR``, else ``NEXRT_LAYERS_DIR``); ``do_sample: false`` means greedy."""
    gen = _generation_config(model_dir or os.environ.get("NEXRT_MODEL_DIR") or os.environ.get("NEXRT_LAYERS_DIR"))
    if gen.get("do_sample") is False:
        return SamplingConfig.make(GREEDY[0], gen.get("top_p", DEFAULT_SAMPLING[1]), GREEDY[2]).as_tuple()
    picked = [gen.get(key, default) for key, default in zip(("temperature", "top_p", "top_k"), DEFAULT_SAMPLING)]
    return SamplingConfig.make(*picked).as_tuple()


def sampling_words(seed, temperature, top_p, top_k) -> List[int]:
    """Eight signed 64-bit words: seed, packed (temperature, top_p), top_k, zeros."""
    return SamplingConfig.make(temperature, top_p, top_k).pack(seed)


# ---- CPU oracle of the device sampler (exact integer RNG, float32 arithmetic) ----------------
_MASK64 = (1 << 64) - 1


def splitmix64(value: int) -> int:
    value = (value + 0x9E3779B97F4A7C15) & _MASK64
    value = ((value ^ (value >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    value = ((value ^ (value >> 27)) * 0x94D049BB133111EB) & _MASK64
    return value ^ (value >> 31)


def seeded_uniform(seed: int, position: int) -> float:
    """Uniform in [0, 1) for an absolute position: top 24 bits of hash(seed, position)."""
    hashed = splitmix64((seed & _MASK64) ^ splitmix64(position & 0xFFFFFFFF))
    return (hashed >> 40) / 16777216.0


def sample_reference(logits, seed, position, temperature, top_p, top_k):
    """Float64 reference of top-k / temperature / top-p sampling.  Returns
    ``(token, kept_ids, kept_probs)``; ties in the top-k go to the lowest token id."""
    import numpy as np

    lg = np.asarray(logits, dtype=np.float64)
    order = np.lexsort((np.arange(lg.size), -lg))[:top_k]
    if temperature == 0.0 or top_k == 1:
        return int(order[0]), [int(order[0])], [1.0]
    p = np.exp((lg[order] - lg[order[0]]) / temperature)
    p /= p.sum()
    cum = np.cumsum(p)
    kept = int(np.searchsorted(cum, top_p - 1e-12) + 1)
    kept = min(max(kept, 1), top_k)
    q = p[:kept] / p[:kept].sum()
    u = seeded_uniform(seed, position)
    idx = int(np.searchsorted(np.cumsum(q), u))
    idx = min(idx, kept - 1)
    return int(order[idx]), [int(i) for i in order[:kept]], q.tolist()
