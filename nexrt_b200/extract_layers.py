"""Split a Hugging Face sharded checkpoint into the per-layer files the loader reads.

Output layout (same file names as the reference's ``tools/extract_layers.py:47-130``):
``layer.<L>.safetensors`` for every decoder layer, ``embed_tokens.safetensors``, ``norm.safetensors``,
``lm_head.safetensors`` and, when the source carries ``mtp.*`` tensors, ``mtp.safetensors``.  Scale
tensors are written in fp32 under ``*.weight_scale_inv`` whichever of the two names the source uses.
The source is read shard by shard through ``model.safetensors.index.json`` so peak host memory is one
layer.

    python -m nexrt_b200.extract_layers --src /ckpt/Nex-N2.5-Pro --dst /data/nexrt-layers [--layers 0 1 2]
"""

from __future__ import annotations

import argparse
import json
import os
import time
from typing import Dict, Iterable, List, Optional

from .config import full_config
from .weights import PFX

GLOBAL_FILES = {"embed_tokens.safetensors": PFX + "embed_tokens.weight", "norm.safetensors": PFX + "norm.weight", "lm_head.safetensors": "lm_head.weight"}


def canonical_key(key: str) -> str:
    return key + "_inv" if key.endswith(".weight_scale") else key


def plan_outputs(weight_map: Dict[str, str], layers: Iterable[int], with_globals: bool = True, with_mtp: bool = True) -> Dict[str, List[str]]:
    """``{output file: [source keys]}``; raises ``KeyError`` for a layer or global tensor the source lacks."""
    out: Dict[str, List[str]] = {}
    for L in layers:
        pref = f"{PFX}layers.{L}."
        keys = sorted(k for k in weight_map if k.startswith(pref))
        if not keys:
            raise KeyError(f"no tensors for layer {L} in the source index")
        out[f"layer.{L}.safetensors"] = keys
    if with_globals:
        for name, key in GLOBAL_FILES.items():
            if key not in weight_map:
                raise KeyError(f"required tensor {key} missing from the source index")
            out[name] = [key]
    mtp = sorted(k for k in weight_map if k.startswith("mtp."))
    if with_mtp and mtp:
        out["mtp.safetensors"] = mtp
    return out


def _write_group(src: str, dst: str, name: str, keys: List[str], weight_map: Dict[str, str], log, t0: float) -> int:
    """One output file: the tensors ``keys`` of the sharded source under their canonical names (scales in fp32), written
    beside its final name and renamed into place."""
    from safetensors import safe_open
    from safetensors.torch import save_file

    by_shard: Dict[str, List[str]] = {}
    for k in keys:
        by_shard.setdefault(weight_map[k], []).append(k)
    tensors = {}
    for shard, ks in sorted(by_shard.items()):
        with safe_open(os.path.join(src, shard), framework="pt", device="cpu") as f:
            for k in ks:
                ck = canonical_key(k)
                if ck in tensors and ck != k:
                    continue                      # both spellings present: keep the first
                t = f.get_tensor(k)
                tensors[ck] = t.float() if ck.endswith(".weight_scale_inv") else t
    tmp = os.path.join(dst, name + f".{os.getpid()}.tmp")
    save_file(tensors, tmp)
    os.replace(tmp, os.path.join(dst, name))
    log(f"  wrote {name}: {len(tensors)} tensors, {sum(v.numel() * v.element_size() for v in tensors.values()) / 1e9:.2f} GB (t={time.time() - t0:.1f}s)")
    return len(tensors)


def _weight_map(src: str) -> Dict[str, str]:
    with open(os.path.join(src, "model.safetensors.index.json"), encoding="utf-8") as f:
        return json.load(f)["weight_map"]


def extract(src: Optional[str], dst: str, layers: Optional[Iterable[int]] = None, with_globals: bool = True, with_mtp: bool = True, log=print,
            mtp_src: Optional[str] = None) -> Dict[str, int]:
    """Split the sharded checkpoint ``src`` into per-layer files under ``dst``.  ``mtp_src`` names a second sharded
    checkpoint whose ``mtp.*`` tensors (and nothing else of it) become ``mtp.safetensors`` - the MTP head is published
    apart from the target (reference tools/extract_layers.py:123-152); with ``src=None`` only that file is written."""
    os.makedirs(dst, exist_ok=True)
    written, t0 = {}, time.time()
    if src is not None:
        weight_map = _weight_map(src)
        n_layers = full_config().n_layers
        layers = range(n_layers) if layers is None else list(layers)
        targets = plan_outputs(weight_map, layers, with_globals, with_mtp and mtp_src is None)
        for name, keys in targets.items():
            written[name] = _write_group(src, dst, name, keys, weight_map, log, t0)
    if mtp_src is not None:
        mtp_map = _weight_map(mtp_src)
        keys = sorted(k for k in mtp_map if k.startswith("mtp."))
        if not keys:
            raise KeyError(f"no mtp.* tensors in {mtp_src}")
        written["mtp.safetensors"] = _write_group(mtp_src, dst, "mtp.safetensors", keys, mtp_map, log, t0)
    return written


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--src", default=os.environ.get("NEXRT_MODEL_DIR"),
                    help="sharded target checkpoint (default NEXRT_MODEL_DIR; omit both to write mtp.safetensors only)")
    ap.add_argument("--mtp-src", default=os.environ.get("NEXRT_MTP_MODEL_DIR"),
                    help="sharded checkpoint whose mtp.* tensors become mtp.safetensors (default NEXRT_MTP_MODEL_DIR; may be the target checkpoint itself)")
    ap.add_argument("--dst", default=os.environ.get("NEXRT_LAYERS_DIR"))
    ap.add_argument("--layers", type=int, nargs="*", default=None)
    ap.add_argument("--no-globals", action="store_true")
    ap.add_argument("--no-mtp", action="store_true")
    a = ap.parse_args(argv)
    if not a.dst:
        ap.error("--dst or NEXRT_LAYERS_DIR is required")
    if not a.src and not a.mtp_src:
        ap.error("--src or --mtp-src is required")
    extract(a.src, a.dst, a.layers, not a.no_globals, not a.no_mtp, mtp_src=a.mtp_src)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
