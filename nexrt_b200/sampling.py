"""Sampling parameters and the fixed 64-byte device buffer they travel in.

Same contract as the reference (``nex_n2_5_pro/sampling.py:30-81``): ``uint64[8]`` =
``[seed, (f32 temperature | f32 top_p), top_k, 5 reserved]``, ``top_k <= 28``, defaults
``(0.6, 0.95, 20)`` overridable by a ``generation_config.json`` next to the weights.  Parameters
live in device memory so a captured graph never needs recapture when a request changes them.
"""

from __future__ import annotations

import json
import math
import operator
import os
import struct
from pathlib import Path

MAX_TOP_K = 28
SAMPLING_WORDS = 8
DEFAULT_SAMPLING = (0.6, 0.95, 20)
GREEDY = (0.0, 1.0, 1)


def checked_sampling_config(temperature, top_p, top_k):
    """Validate and return the values exactly as the device will see them (float32 rounded)."""
    temperature, top_p = float(temperature), float(top_p)
    if not math.isfinite(temperature) or temperature < 0:
        raise ValueError("temperature must be finite and >= 0")
    if not math.isfinite(top_p) or not 0 < top_p <= 1:
        raise ValueError("top_p must be finite and in (0, 1]")
    if isinstance(top_k, bool):
        raise ValueError(f"top_k must be an integer in [1, {MAX_TOP_K}]")
    try:
        top_k = operator.index(top_k)
    except TypeError as error:
        raise ValueError(f"top_k must be an integer in [1, {MAX_TOP_K}]") from error
    if not 1 <= top_k <= MAX_TOP_K:
        raise ValueError(f"top_k must be in [1, {MAX_TOP_K}]")
    try:
        t32, p32 = struct.unpack("<ff", struct.pack("<ff", temperature, top_p))
    except (OverflowError, struct.error) as error:
        raise ValueError("sampling parameters must fit float32") from error
    if (temperature > 0 and t32 == 0) or p32 == 0:
        raise ValueError("sampling parameters must not underflow float32")
    return t32, p32, top_k


def resolve_sampling_config(defaults, temperature=None, top_p=None, top_k=None):
    given = (temperature, top_p, top_k)
    return checked_sampling_config(*(d if g is None else g for d, g in zip(defaults, given)))


def sampling_defaults():
    model_dir = os.environ.get("NEXRT_MODEL_DIR") or os.environ.get("NEXRT_LAYERS_DIR")
    config = {}
    if model_dir:
        path = Path(model_dir) / "generation_config.json"
        if path.is_file():
            config = json.loads(path.read_text())
    temperature = config.get("temperature", DEFAULT_SAMPLING[0])
    top_p = config.get("top_p", DEFAULT_SAMPLING[1])
    top_k = config.get("top_k", DEFAULT_SAMPLING[2])
    if config.get("do_sample") is False:
        temperature, top_k = 0.0, 1
    return checked_sampling_config(temperature, top_p, top_k)


def sampling_words(seed, temperature, top_p, top_k):
    """Eight signed 64-bit words: seed, packed (temperature, top_p), top_k, zeros."""
    temperature, top_p, top_k = checked_sampling_config(temperature, top_p, top_k)
    seed = int(seed) & ((1 << 64) - 1)
    signed_seed = seed if seed < (1 << 63) else seed - (1 << 64)
    packed = struct.unpack("<q", struct.pack("<ff", temperature, top_p))[0]
    return [signed_seed, packed, top_k] + [0] * (SAMPLING_WORDS - 3)


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
