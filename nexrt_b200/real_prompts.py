"""Deterministic prompts of an exact token length.

``build_real_prompt(L, tok)`` returns exactly ``L`` ids: long-form text wrapped in the tokenizer's
chat template with the document cropped in the middle, so the generation-prompt tail is always intact
(behaviour of the reference's ``real_prompts.py:94-125``).  Text comes from ``data_en/*.jsonl``
(``{"content": ...}`` per line, produced by :mod:`nexrt_b200.prep_english_docs`); when no corpus is
installed a fixed built-in paragraph is tiled, which keeps the function usable offline.
``synthetic`` prompts for benchmarks live in :func:`nexrt_b200.models.reference.synthetic_prompt`.
"""

from __future__ import annotations

import glob
import json
import os
from typing import List

_DOC_GLOB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data_en", "*.jsonl")
_FALLBACK = (
    "A decode engine spends most of its time waiting: for weights to arrive from memory, for a peer to publish a partial sum, "
    "for the host to notice that a token is ready. Making it fast is the craft of removing those waits one by one, and of proving, "
    "after each removal, that the answer did not change. "
)
_pool = {"text": "", "chars": 0}


def text_pool(min_chars: int) -> str:
    if _pool["chars"] >= min_chars:
        return _pool["text"]
    parts, total = [], 0
    for path in sorted(glob.glob(_DOC_GLOB)):
        with open(path, encoding="utf-8") as f:
            for line in f:
                try:
                    content = json.loads(line).get("content", "").strip()
                except (json.JSONDecodeError, AttributeError):
                    continue
                if content:
                    parts.append(content)
                    total += len(content) + 2
                    if total >= min_chars:
                        break
        if total >= min_chars:
            break
    if total < min_chars:
        base = "\n\n".join(parts) or _FALLBACK
        parts = [base] * (min_chars // len(base) + 1)
    _pool["text"] = "\n\n".join(parts)
    _pool["chars"] = len(_pool["text"])
    return _pool["text"]


def _ids(enc) -> List[int]:
    ids = enc if isinstance(enc, list) else enc["input_ids"]
    if ids and isinstance(ids[0], list):
        ids = ids[0]
    return [int(t) for t in ids]


def fixed_suffix_len(tok) -> int:
    """Number of trailing tokens every templated user prompt shares (turn close + generation prompt)."""
    a = _ids(tok.apply_chat_template([{"role": "user", "content": "a"}], add_generation_prompt=True, tokenize=True))
    b = _ids(tok.apply_chat_template([{"role": "user", "content": "bb bb"}], add_generation_prompt=True, tokenize=True))
    n = 0
    while n < min(len(a), len(b)) and a[-1 - n] == b[-1 - n]:
        n += 1
    return max(1, n)


def build_real_prompt(L: int, tok) -> List[int]:
    if L < 8:
        raise ValueError("L is too small for a chat-templated prompt")
    tail = fixed_suffix_len(tok)
    if L <= tail:
        raise ValueError(f"L={L} does not leave room for the {tail}-token template tail")
    chars, ids = max(64, 5 * L), []
    for _ in range(12):
        ids = _ids(tok.apply_chat_template([{"role": "user", "content": text_pool(chars)[:chars]}], add_generation_prompt=True, tokenize=True))
        if len(ids) >= L:
            break
        chars *= 2
    if len(ids) < L:
        raise ValueError(f"could not reach {L} tokens (got {len(ids)})")
    ids = ids[: L - tail] + ids[-tail:]
    assert len(ids) == L
    return ids
