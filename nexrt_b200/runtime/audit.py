"""Memory-safety audits that need no sanitizer: guard bands around scratch buffers and a pointer-disjointness check.

``compute-sanitizer`` is not available where this framework is developed, so the two classes of bug it would catch in
the step kernels are checked from the host instead:

* **out-of-bounds writes** - with ``NEXRT_CANARY=1`` every scratch buffer of a ``StepContext`` is carved out of its own
  arena with a 256-byte band of a known pattern before and after it (and over the padding up to the next 256 bytes);
  ``violated()`` names the buffers whose bands changed.  A kernel that writes row ``M`` of an ``M``-row buffer, or one
  element past a ragged tile, lands in a band instead of in a neighbour's data.
* **aliasing** - ``overlaps()`` takes every tensor an engine holds (context scratch, caches, rings, weights) and reports
  pairs whose byte ranges intersect although they do not share one storage object on purpose.

The reference guards its 8-row CP exchange with canary words checked by ``cp_guard_ok``
(``nex_n2_5_pro/m8_cp.py:80-500``); this is the same idea applied to every scratch buffer of the engine.
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Sequence, Tuple

import torch

GUARD_BYTES = 256
PATTERN = 0xA5


def guarded_zeros(registry: List, shape: Sequence[int], dtype: torch.dtype, device) -> torch.Tensor:
    """A zero tensor of ``shape`` inside its own arena ``[guard | data | pad | guard]``; the arena goes into ``registry``."""
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    padded = (nbytes + GUARD_BYTES - 1) // GUARD_BYTES * GUARD_BYTES
    arena = torch.full((GUARD_BYTES + padded + GUARD_BYTES,), PATTERN, dtype=torch.uint8, device=device)
    body = arena[GUARD_BYTES : GUARD_BYTES + nbytes]
    body.zero_()
    registry.append((arena, nbytes))
    return body.view(dtype).view(*shape)


def violated(registry: Iterable[Tuple[torch.Tensor, int]]) -> List[int]:
    """Indices (allocation order) of the arenas whose guard bands or padding no longer hold the pattern."""
    bad = []
    for i, (arena, nbytes) in enumerate(registry):
        front = arena[:GUARD_BYTES]
        back = arena[GUARD_BYTES + nbytes :]
        if bool((front != PATTERN).any()) or bool((back != PATTERN).any()):
            bad.append(i)
    return bad


def named_tensors(obj, prefix: str = "", depth: int = 3, seen=None) -> Dict[str, torch.Tensor]:
    """Every tensor reachable from ``obj`` through attributes, lists, tuples and dicts (a few levels deep)."""
    seen = set() if seen is None else seen
    out: Dict[str, torch.Tensor] = {}
    if id(obj) in seen or depth < 0:
        return out
    seen.add(id(obj))
    if isinstance(obj, torch.Tensor):
        out[prefix or "tensor"] = obj
        return out
    if isinstance(obj, dict):
        items = obj.items()
    elif isinstance(obj, (list, tuple)):
        items = enumerate(obj)
    elif hasattr(obj, "__dict__"):
        items = vars(obj).items()
    else:
        return out
    for key, value in items:
        name = f"{prefix}.{key}" if prefix else str(key)
        if isinstance(value, torch.Tensor):
            out[name] = value
        elif isinstance(value, (dict, list, tuple)) or (hasattr(value, "__dict__") and not isinstance(value, type) and not callable(value)):
            out.update(named_tensors(value, name, depth - 1, seen))
    return out


def _extent(t: torch.Tensor) -> Tuple[int, int]:
    if t.numel() == 0:
        return (t.data_ptr(), t.data_ptr())
    # bytes spanned by a (possibly strided) view
    span = 1 + sum((s - 1) * abs(st) for s, st in zip(t.shape, t.stride()))
    return (t.data_ptr(), t.data_ptr() + span * t.element_size())


def overlaps(tensors: Dict[str, torch.Tensor]) -> List[Tuple[str, str]]:
    """Pairs of tensors whose byte ranges intersect without sharing a storage (views of one storage are deliberate)."""
    rows = []
    for name, t in tensors.items():
        if t.numel() == 0:
            continue
        lo, hi = _extent(t)
        rows.append((lo, hi, t.untyped_storage().data_ptr(), str(t.device), name))
    rows.sort()
    bad = []
    for i, (lo, hi, storage, dev, name) in enumerate(rows):
        for lo2, hi2, storage2, dev2, name2 in rows[i + 1 :]:
            if lo2 >= hi:
                break
            if dev == dev2 and storage != storage2:
                bad.append((name, name2))
    return bad


def engine_tensors(engine) -> Dict[str, torch.Tensor]:
    """The tensors an engine launches kernels on: context scratch, per-layer caches / rings / weights, head, taps."""
    out = named_tensors(engine.ctx, "ctx")
    for i, m in enumerate(getattr(engine, "mixers", [])):
        out.update(named_tensors(m, f"mixer{i}", depth=2))
    for i, m in enumerate(getattr(engine, "moes", [])):
        out.update(named_tensors(m, f"moe{i}", depth=2))
    out.update(named_tensors(getattr(engine, "head", None), "head", depth=2))
    if getattr(engine, "taps", None) is not None:
        out["taps"] = engine.taps
    return out
