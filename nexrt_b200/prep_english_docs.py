"""Build the ``data_en/*.jsonl`` corpus used by :func:`nexrt_b200.real_prompts.build_real_prompt`.

Input: a ShareGPT-style JSON file (a list of ``{"conversations": [{"from": ..., "value": ...}]}``).
Keeps long, mostly-ASCII assistant turns with fenced code removed and writes ``{"content": ...}`` lines
until ``--target-chars`` characters are collected (what the reference's ``prep_english_docs.py:39-90``
produces).
"""

from __future__ import annotations

import argparse
import json
import re
from pathlib import Path

DEFAULT_OUT = Path(__file__).resolve().parent / "data_en" / "docs.jsonl"
_FENCE = re.compile(r"```.*?```", re.S)


def ascii_fraction(s: str) -> float:
    return sum(1 for c in s if ord(c) < 128) / max(1, len(s))


def clean_turn(text: str, min_chars: int = 400, min_ascii: float = 0.98):
    text = _FENCE.sub("", text or "").strip()
    text = re.sub(r"\n{3,}", "\n\n", text)
    return text if len(text) >= min_chars and ascii_fraction(text) >= min_ascii else None


def collect(records, target_chars: int):
    total = 0
    for rec in records:
        for turn in rec.get("conversations", ()) if isinstance(rec, dict) else ():
            if turn.get("from") not in ("gpt", "assistant"):
                continue
            text = clean_turn(turn.get("value", ""))
            if text:
                yield text
                total += len(text)
                if total >= target_chars:
                    return


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--src", required=True)
    ap.add_argument("--out", type=Path, default=DEFAULT_OUT)
    ap.add_argument("--target-chars", type=int, default=4_000_000)
    a = ap.parse_args(argv)
    with open(a.src, encoding="utf-8") as f:
        records = json.load(f)
    a.out.parent.mkdir(parents=True, exist_ok=True)
    n = chars = 0
    with open(a.out, "w", encoding="utf-8") as f:
        for text in collect(records, a.target_chars):
            f.write(json.dumps({"content": text}, ensure_ascii=False) + "\n")
            n, chars = n + 1, chars + len(text)
    print(f"wrote {n} documents, {chars} characters to {a.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
