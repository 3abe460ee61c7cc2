"""Checkpoint I/O (Hugging Face key layout), random initialisation and tensor-parallel sharding.

Key names and the per-layer file split (``layer.{L}.safetensors``, ``embed_tokens.safetensors``,
``norm.safetensors``, ``lm_head.safetensors``) are the reference's
(``nex_n2_5_pro/weights.py:38-60,66-81,108-126,166-199``); both ``*.weight_scale_inv`` and
``*.weight_scale`` are accepted (``weights.py:27-31``).  Sharding reproduces the reference's
row/column slices (``weights.py:84-105,128-164``; MoE ``moe.py:145-171``) for any
``tp in {1,2,4,8}`` instead of only 8.

The per-rank tensors are packed in the layout the sm_100a kernels stream:

* GDN ``front_w [q|k|v|z rows, H]`` fp8 + ``front_s``; ``ba_w [b rows|a rows, H]`` bf16;
  ``conv_w [qkv rows, 4]`` fp32; ``out_w [H, v_local]`` fp8.
* attention ``front_w [(q|gate) per head, k, v rows, H]`` fp8; ``out_w [H, q_local]`` fp8.
* MoE ``router_w [E+1, H]`` bf16 (row E is the shared-expert gate), ``w13 [E+1, 2I, H]`` fp8
  (gate rows then up rows; index E is the shared expert), ``w2 [E+1, H, I]`` fp8.

RMSNorm multipliers are stored as ``1 + w`` in fp32 and applied to the activation inside the
kernels, so no weight is re-quantised at load (the reference folds them into the fp8 weights,
``gdn.py:83-113``, which perturbs every block scale).
"""

from __future__ import annotations

from pathlib import Path
from typing import Dict, Mapping, Optional

import torch

from .config import BLOCK, ModelConfig, ShardSpec
from .quant import FP8, quantize_blockwise

PFX = "model.language_model."
INIT_STD = 0.02


# --------------------------------------------------------------------------------------------
# random initialisation (global tensors, HF names)
# --------------------------------------------------------------------------------------------
def _randn(gen, *shape, device="cpu"):
    return torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * INIT_STD


def _put_fp8(out, name, w):
    q, s = quantize_blockwise(w)
    out[name + ".weight"] = q
    out[name + ".weight_scale_inv"] = s


def random_layer(cfg: ModelConfig, layer: int, gen, device="cpu") -> Dict[str, torch.Tensor]:
    """One decoder layer's tensors under HF names, drawn N(0, 0.02) then quantised."""
    H, out = cfg.hidden, {}
    p = f"{PFX}layers.{layer}."
    bf = torch.bfloat16
    out[p + "input_layernorm.weight"] = _randn(gen, H, device=device).to(bf)
    out[p + "post_attention_layernorm.weight"] = _randn(gen, H, device=device).to(bf)
    if cfg.layer_types[layer] == "linear":
        a = p + "linear_attn."
        kd, vd, nv = cfg.gdn_key_dim, cfg.gdn_value_dim, cfg.gdn_v_heads
        _put_fp8(out, a + "in_proj_qkv", _randn(gen, 2 * kd + vd, H, device=device))
        _put_fp8(out, a + "in_proj_z", _randn(gen, vd, H, device=device))
        _put_fp8(out, a + "out_proj", _randn(gen, H, vd, device=device))
        out[a + "in_proj_b.weight"] = _randn(gen, nv, H, device=device).to(bf)
        out[a + "in_proj_a.weight"] = _randn(gen, nv, H, device=device).to(bf)
        out[a + "conv1d.weight"] = (
            _randn(gen, 2 * kd + vd, 1, cfg.conv_kernel, device=device) * 10.0
        ).to(bf)
        out[a + "A_log"] = _randn(gen, nv, device=device)
        out[a + "dt_bias"] = _randn(gen, nv, device=device)
        out[a + "norm.weight"] = (1.0 + _randn(gen, cfg.gdn_dim, device=device)).to(bf)
    else:
        a = p + "self_attn."
        hd = cfg.head_dim
        _put_fp8(out, a + "q_proj", _randn(gen, cfg.n_q_heads * 2 * hd, H, device=device))
        _put_fp8(out, a + "k_proj", _randn(gen, cfg.n_kv_heads * hd, H, device=device))
        _put_fp8(out, a + "v_proj", _randn(gen, cfg.n_kv_heads * hd, H, device=device))
        _put_fp8(out, a + "o_proj", _randn(gen, H, cfg.n_q_heads * hd, device=device))
        out[a + "q_norm.weight"] = _randn(gen, hd, device=device).to(bf)
        out[a + "k_norm.weight"] = _randn(gen, hd, device=device).to(bf)
    m = p + "mlp."
    out[m + "gate.weight"] = _randn(gen, cfg.n_experts, H, device=device).to(bf)
    out[m + "shared_expert_gate.weight"] = _randn(gen, 1, H, device=device).to(bf)
    I = cfg.moe_inter
    for e in list(range(cfg.n_experts)) + ["shared"]:
        ep = m + ("shared_expert." if e == "shared" else f"experts.{e}.")
        _put_fp8(out, ep + "gate_proj", _randn(gen, I, H, device=device))
        _put_fp8(out, ep + "up_proj", _randn(gen, I, H, device=device))
        _put_fp8(out, ep + "down_proj", _randn(gen, H, I, device=device))
    return out


def random_checkpoint(cfg: ModelConfig, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    """Whole model under HF names (small geometries only: everything is materialised)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    out = {
        PFX + "embed_tokens.weight": _randn(gen, cfg.vocab, cfg.hidden, device=device).to(torch.bfloat16),
        PFX + "norm.weight": _randn(gen, cfg.hidden, device=device).to(torch.bfloat16),
        "lm_head.weight": _randn(gen, cfg.vocab, cfg.hidden, device=device).to(torch.bfloat16),
    }
    for layer in range(cfg.n_layers):
        out.update(random_layer(cfg, layer, gen, device))
    return out


# --------------------------------------------------------------------------------------------
# safetensors layout
# --------------------------------------------------------------------------------------------
def save_checkpoint(ckpt: Dict[str, torch.Tensor], cfg: ModelConfig, out_dir) -> None:
    from safetensors.torch import save_file

    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    cpu = {k: v.detach().cpu().contiguous() for k, v in ckpt.items()}
    save_file({k: cpu[k] for k in (PFX + "embed_tokens.weight",)}, str(out_dir / "embed_tokens.safetensors"))
    save_file({PFX + "norm.weight": cpu[PFX + "norm.weight"]}, str(out_dir / "norm.safetensors"))
    save_file({"lm_head.weight": cpu["lm_head.weight"]}, str(out_dir / "lm_head.safetensors"))
    for layer in range(cfg.n_layers):
        p = f"{PFX}layers.{layer}."
        save_file({k: v for k, v in cpu.items() if k.startswith(p)}, str(out_dir / f"layer.{layer}.safetensors"))
    extra = {k: v for k, v in cpu.items() if k.startswith("mtp.")}
    if extra:
        save_file(extra, str(out_dir / "mtp.safetensors"))


def _scale_key(keys, key):
    """Accept both checkpoint names of the dequantisation multiplier."""
    if key in keys:
        return key
    alt = key[: -len("_inv")] if key.endswith("_inv") else key + "_inv"
    if alt in keys:
        return alt
    raise KeyError(key)


def load_checkpoint(cfg: ModelConfig, layers_dir, device="cpu") -> Dict[str, torch.Tensor]:
    """Read every file of a layer directory back into one HF-named dict."""
    from safetensors import safe_open

    out = {}
    names = ["embed_tokens", "norm", "lm_head"] + [f"layer.{l}" for l in range(cfg.n_layers)]
    if (Path(layers_dir) / "mtp.safetensors").is_file():
        names.append("mtp")
    for name in names:
        with safe_open(str(Path(layers_dir) / f"{name}.safetensors"), framework="pt", device=str(device)) as f:
            for k in f.keys():
                out[k] = f.get_tensor(k)
    return out


def prefault_file(path) -> int:
    """Read ``path`` once, front to back, so that the page cache holds it when the loader maps it (a cold 7 GB layer file
    otherwise faults in 4 KB at a time under the tensor copies).  Strictly read-only: the file is opened ``O_RDONLY``,
    nothing is written beside it, and its times are left alone where the platform allows (``O_NOATIME`` when permitted).
    Returns the number of bytes read.  The reference warms checkpoint files the same way before SGLang maps them
    (``sglang_prefill/weight_loading.py``: ``_prefault_checkpoint_file``)."""
    import os

    flags = os.O_RDONLY | getattr(os, "O_CLOEXEC", 0)
    try:
        fd = os.open(str(path), flags | getattr(os, "O_NOATIME", 0))
    except PermissionError:          # O_NOATIME needs ownership of the file
        fd = os.open(str(path), flags)
    total = 0
    try:
        if hasattr(os, "posix_fadvise"):
            os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_SEQUENTIAL)
        while True:
            chunk = os.read(fd, 16 << 20)
            if not chunk:
                break
            total += len(chunk)
    finally:
        os.close(fd)
    return total


class TensorFiles(Mapping):
    """A list of safetensors files as a read-only mapping ``key -> tensor`` that never holds more than one tensor on the host.

    The files' headers are indexed at construction (names only, no data); a tensor is read when it is asked for and no
    reference to it is kept; the file that was read last stays open, and while it is in use a background thread warms the
    page cache with the next file of the list (``prefault=True``).  ``shape(key)`` answers from the header alone."""

    def __init__(self, paths, device="cpu", prefault: bool = True):
        from safetensors import safe_open

        self.files = [Path(p) for p in paths]
        self.device, self.prefault = str(device), prefault
        self.index: Dict[str, int] = {}
        for i, path in enumerate(self.files):
            with safe_open(str(path), framework="pt", device="cpu") as f:
                for k in f.keys():
                    self.index[k] = i
        self._open_idx, self._open, self._ctx = -1, None, None
        self._warm = None                   # thread warming the page cache with file self._warmed
        self._warmed = -1
        self.reads = 0                      # tensors read so far

    # ---- Mapping ----
    def __len__(self) -> int:
        return len(self.index)

    def __iter__(self):
        return iter(self.index)

    def __contains__(self, key) -> bool:
        return key in self.index

    def __getitem__(self, key: str) -> torch.Tensor:
        self._use(self.index[key])          # KeyError for an unknown name, like a dict
        self.reads += 1
        return self._open.get_tensor(key)

    def shape(self, key: str):
        """Shape of ``key`` from its file's header (no tensor data is read)."""
        self._use(self.index[key])
        return tuple(self._open.get_slice(key).get_shape())

    # ---- files ----
    def _use(self, i: int) -> None:
        if i == self._open_idx:
            return
        from safetensors import safe_open

        self.close()
        if self._warm is not None and self._warmed == i:
            self._warm.join()               # the file being opened is the one being warmed: let the read finish
        self._ctx = safe_open(str(self.files[i]), framework="pt", device=self.device)
        self._open = self._ctx.__enter__()
        self._open_idx = i
        nxt = i + 1
        if self.prefault and nxt < len(self.files) and nxt > self._warmed:
            import threading

            self._warmed = nxt
            self._warm = threading.Thread(target=prefault_file, args=(self.files[nxt],), daemon=True)
            self._warm.start()

    def close(self) -> None:
        if self._ctx is not None:
            self._ctx.__exit__(None, None, None)
        self._ctx, self._open, self._open_idx = None, None, -1


class LayerFiles(TensorFiles):
    """A layer directory (``embed_tokens``, ``norm``, ``lm_head``, ``layer.{L}``, optionally ``mtp``) as one mapping.

    ``load_checkpoint`` materialises every file of the directory in one dict, which for the full model is the whole
    checkpoint in host memory on every rank.  The sharding functions only ever ask for one key at a time (and for
    ``keys()`` when a scale goes by either of its two names), so ``shard_model(LayerFiles(cfg, dir), ...)`` streams the
    directory once, in file order, with a host footprint of one tensor and the next layer's file warming behind it
    (reference: per-layer files read one layer at a time, ``weights.py:166-199``)."""

    def __init__(self, cfg: ModelConfig, layers_dir, device="cpu", prefault: bool = True):
        root = Path(layers_dir)
        names = ["embed_tokens", "norm", "lm_head"] + [f"layer.{l}" for l in range(cfg.n_layers)]
        if (root / "mtp.safetensors").is_file():
            names.append("mtp")
        super().__init__([root / f"{n}.safetensors" for n in names], device=device, prefault=prefault)
        self.dir = root


def load_rank_model(cfg: ModelConfig, layers_dir, tp: int, rank: int, device, cp: bool = False, prefault: bool = True) -> Dict:
    """One rank's kernel-layout tensors straight from a layer directory, one tensor on the host at a time."""
    files = LayerFiles(cfg, layers_dir, prefault=prefault)
    try:
        return shard_model(files, cfg, tp, rank, device, cp=cp)
    finally:
        files.close()


def normalise_scale_names(ckpt: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Rename ``*.weight_scale`` to ``*.weight_scale_inv`` (reference tools/extract_layers.py:103-109)."""
    out = {}
    for k, v in ckpt.items():
        out[k + "_inv" if k.endswith(".weight_scale") else k] = v
    return out


# --------------------------------------------------------------------------------------------
# sharding into the kernel layout
# --------------------------------------------------------------------------------------------
def _g(ckpt, key):
    if key.endswith("weight_scale_inv"):
        key = _scale_key(ckpt.keys(), key)
    return ckpt[key]


def _gamma(w: torch.Tensor) -> torch.Tensor:
    """Gemma-style RMSNorm multiplier ``1 + w`` in fp32 (reference attn.py:102-105)."""
    return (1.0 + w.float()).contiguous()


def _rows(t, start, count):
    return t[start : start + count]


def shard_linear_attention(ckpt, cfg: ModelConfig, layer: int, spec: ShardSpec, device) -> Dict[str, torch.Tensor]:
    """GDN shard: ``q|k|v|z`` rows of this rank's heads (reference weights.py:128-164)."""
    a = f"{PFX}layers.{layer}.linear_attn."
    D, tp, r = cfg.gdn_dim, spec.tp, spec.rank
    kd, vd = cfg.gdn_key_dim, cfg.gdn_value_dim
    kr, vr = kd // tp, vd // tp
    qkv, qkvs = _g(ckpt, a + "in_proj_qkv.weight"), _g(ckpt, a + "in_proj_qkv.weight_scale_inv").float()
    z, zs = _g(ckpt, a + "in_proj_z.weight"), _g(ckpt, a + "in_proj_z.weight_scale_inv").float()

    def gather(t, unit):
        return [
            _rows(t, r * kr // unit, kr // unit),
            _rows(t, (kd + r * kr) // unit, kr // unit),
            _rows(t, (2 * kd + r * vr) // unit, vr // unit),
        ]

    front_w = torch.cat(gather(qkv.view(torch.uint8), 1) + [_rows(z.view(torch.uint8), r * vr, vr)], 0)
    front_s = torch.cat(gather(qkvs, BLOCK) + [_rows(zs, r * vr // BLOCK, vr // BLOCK)], 0)
    conv = _g(ckpt, a + "conv1d.weight").float().reshape(2 * kd + vd, cfg.conv_kernel)
    o, os_ = _g(ckpt, a + "out_proj.weight"), _g(ckpt, a + "out_proj.weight_scale_inv").float()
    nv = spec.gdn_v
    ba = torch.cat(
        [_rows(_g(ckpt, a + "in_proj_b.weight"), r * nv, nv), _rows(_g(ckpt, a + "in_proj_a.weight"), r * nv, nv)], 0
    )
    d = lambda t: t.contiguous().to(device)
    return {
        "kind": "linear",
        "in_ln": d(_gamma(ckpt[f"{PFX}layers.{layer}.input_layernorm.weight"])),
        "front_w": d(front_w).view(FP8),
        "front_s": d(front_s),
        "ba_w": d(ba.to(torch.bfloat16)),
        "conv_w": d(torch.cat(gather(conv, 1), 0)),
        "a_log": d(_rows(_g(ckpt, a + "A_log").float(), r * nv, nv)),
        "dt_bias": d(_rows(_g(ckpt, a + "dt_bias").float(), r * nv, nv)),
        "gnorm_w": d(_g(ckpt, a + "norm.weight").float()),
        "out_w": d(o.view(torch.uint8)[:, r * vr : (r + 1) * vr]).view(FP8),
        "out_s": d(os_[:, r * vr // BLOCK : (r + 1) * vr // BLOCK]),
    }


def shard_attention(ckpt, cfg: ModelConfig, layer: int, spec: ShardSpec, device, base: Optional[str] = None) -> Dict[str, torch.Tensor]:
    """Attention shard: this rank's q heads (query|gate interleaved per head) plus the kv head(s)
    it serves (reference weights.py:84-105)."""
    base = base or f"{PFX}layers.{layer}."
    a = base + "self_attn."
    hd, r = cfg.head_dim, spec.rank
    qrows = spec.q_heads * 2 * hd
    kvrows = spec.kv_heads * hd
    kv0 = spec.kv_head0 * hd
    u8 = lambda k: _g(ckpt, a + k).view(torch.uint8)
    sc = lambda k: _g(ckpt, a + k + "_scale_inv").float()
    front_w = torch.cat(
        [_rows(u8("q_proj.weight"), r * qrows, qrows), _rows(u8("k_proj.weight"), kv0, kvrows), _rows(u8("v_proj.weight"), kv0, kvrows)], 0
    )
    front_s = torch.cat(
        [
            _rows(sc("q_proj.weight"), r * qrows // BLOCK, qrows // BLOCK),
            _rows(sc("k_proj.weight"), kv0 // BLOCK, kvrows // BLOCK),
            _rows(sc("v_proj.weight"), kv0 // BLOCK, kvrows // BLOCK),
        ],
        0,
    )
    oc = spec.q_heads * hd
    d = lambda t: t.contiguous().to(device)
    return {
        "kind": "full",
        "in_ln": d(_gamma(ckpt[base + "input_layernorm.weight"])),
        "front_w": d(front_w).view(FP8),
        "front_s": d(front_s),
        "qn": d(_gamma(_g(ckpt, a + "q_norm.weight"))),
        "kn": d(_gamma(_g(ckpt, a + "k_norm.weight"))),
        "out_w": d(u8("o_proj.weight")[:, r * oc : (r + 1) * oc]).view(FP8),
        "out_s": d(sc("o_proj.weight")[:, r * oc // BLOCK : (r + 1) * oc // BLOCK]),
    }


def shard_attention_cp(ckpt, cfg: ModelConfig, layer: int, spec: ShardSpec, device, base: Optional[str] = None) -> Dict[str, torch.Tensor]:
    """Context-parallel front of one rank: the query rows of EVERY q head that shares this rank's kv
    head (the whole cp group's heads, in global head order), then the gate rows of the rank's own
    heads, then k and v (the reference's duplicate-Q weights, attn.py:220-257)."""
    base = base or f"{PFX}layers.{layer}."
    a = base + "self_attn."
    hd = cfg.head_dim
    qw = _g(ckpt, a + "q_proj.weight").view(torch.uint8)
    qs = _g(ckpt, a + "q_proj.weight_scale_inv").float()
    g0 = spec.cp_group[0] * spec.q_heads                      # first global q head of the group
    n_all = spec.q_heads * spec.cp_size
    hb = hd // BLOCK
    rows, scales = [], []
    for h in range(g0, g0 + n_all):                           # query halves
        rows.append(qw[h * 2 * hd : h * 2 * hd + hd]); scales.append(qs[h * 2 * hb : h * 2 * hb + hb])
    for h in range(spec.rank * spec.q_heads, (spec.rank + 1) * spec.q_heads):   # own gate halves
        rows.append(qw[h * 2 * hd + hd : (h + 1) * 2 * hd]); scales.append(qs[h * 2 * hb + hb : (h + 1) * 2 * hb])
    kv0, kvrows = spec.kv_head0 * hd, spec.kv_heads * hd
    for nm in ("k_proj", "v_proj"):
        rows.append(_g(ckpt, a + nm + ".weight").view(torch.uint8)[kv0 : kv0 + kvrows])
        scales.append(_g(ckpt, a + nm + ".weight_scale_inv").float()[kv0 // BLOCK : (kv0 + kvrows) // BLOCK])
    d = lambda t: t.contiguous().to(device)
    return {"front_w": d(torch.cat(rows, 0)).view(FP8), "front_s": d(torch.cat(scales, 0))}


def shard_moe(ckpt, cfg: ModelConfig, layer: int, spec: ShardSpec, device, base: Optional[str] = None) -> Dict[str, torch.Tensor]:
    """MoE shard: every expert, ``inter/tp`` of its intermediate columns (reference moe.py:145-171);
    the shared expert is stored as expert index ``n_experts``."""
    base = base or f"{PFX}layers.{layer}."
    m = base + "mlp."
    E, I, Il, r, H = cfg.n_experts, cfg.moe_inter, spec.inter, spec.rank, cfg.hidden
    w13 = torch.empty(E + 1, 2 * Il, H, dtype=torch.uint8)
    w13s = torch.empty(E + 1, 2 * Il // BLOCK, H // BLOCK, dtype=torch.float32)
    w2 = torch.empty(E + 1, H, Il, dtype=torch.uint8)
    w2s = torch.empty(E + 1, H // BLOCK, Il // BLOCK, dtype=torch.float32)
    nb = Il // BLOCK
    for e in range(E + 1):
        ep = m + ("shared_expert." if e == E else f"experts.{e}.")
        for j, nm in enumerate(("gate_proj", "up_proj")):
            w13[e, j * Il : (j + 1) * Il] = _g(ckpt, ep + nm + ".weight").view(torch.uint8)[r * Il : (r + 1) * Il].cpu()
            w13s[e, j * nb : (j + 1) * nb] = _g(ckpt, ep + nm + ".weight_scale_inv").float()[r * nb : (r + 1) * nb].cpu()
        w2[e] = _g(ckpt, ep + "down_proj.weight").view(torch.uint8)[:, r * Il : (r + 1) * Il].cpu()
        w2s[e] = _g(ckpt, ep + "down_proj.weight_scale_inv").float()[:, r * nb : (r + 1) * nb].cpu()
    router = torch.cat([_g(ckpt, m + "gate.weight"), _g(ckpt, m + "shared_expert_gate.weight").reshape(1, H)], 0)
    d = lambda t: t.contiguous().to(device)
    return {
        "post_ln": d(_gamma(ckpt[base + "post_attention_layernorm.weight"])),
        "router_w": d(router.to(torch.bfloat16)),
        "w13": d(w13).view(FP8),
        "w13_s": d(w13s),
        "w2": d(w2).view(FP8),
        "w2_s": d(w2s),
    }


def shard_head(ckpt, cfg: ModelConfig, spec: ShardSpec, device) -> Dict[str, torch.Tensor]:
    """Vocab-parallel LM-head rows, replicated embedding and final norm (reference head.py:19-25)."""
    V = spec.vocab
    d = lambda t: t.contiguous().to(device)
    return {
        "embed": d(ckpt[PFX + "embed_tokens.weight"].to(torch.bfloat16)),
        "final_ln": d(_gamma(ckpt[PFX + "norm.weight"])),
        "lm_head": d(ckpt["lm_head.weight"][spec.rank * V : (spec.rank + 1) * V].to(torch.bfloat16)),
    }


def shard_model(ckpt, cfg: ModelConfig, tp: int, rank: int, device, cp: bool = False) -> Dict:
    """All tensors one rank needs, in kernel layout.  ``cp`` adds the context-parallel attention
    fronts (``mixer_cp``) when the rank shares its kv head with other ranks."""
    spec = ShardSpec(cfg, tp, rank)
    layers = []
    for layer in range(cfg.n_layers):
        entry = {}
        if cfg.layer_types[layer] == "linear":
            mix = shard_linear_attention(ckpt, cfg, layer, spec, device)
        else:
            mix = shard_attention(ckpt, cfg, layer, spec, device)
            if cp and spec.cp_size > 1:
                entry["mixer_cp"] = shard_attention_cp(ckpt, cfg, layer, spec, device)
        entry.update(mixer=mix, moe=shard_moe(ckpt, cfg, layer, spec, device))
        layers.append(entry)
    return {"spec": spec, "layers": layers, "head": shard_head(ckpt, cfg, spec, device)}


# --------------------------------------------------------------------------------------------
# direct per-rank random initialisation (full geometry: nothing global is ever materialised)
# --------------------------------------------------------------------------------------------
def _rand_fp8(gen, shape, device, chunk_rows=None):
    """N(0, 0.02) weights quantised with 128x128 blocks, generated in bounded fp32 chunks."""
    *lead, R, C = shape
    n_lead = 1
    for v in lead:
        n_lead *= v
    q = torch.empty(n_lead, R, C, dtype=FP8, device=device)
    s = torch.empty(n_lead, R // BLOCK, C // BLOCK, dtype=torch.float32, device=device)
    step = max(1, (1 << 26) // (R * C))  # <= 64 Mi fp32 elements per chunk
    for i in range(0, n_lead, step):
        n = min(step, n_lead - i)
        w = torch.randn(n, R, C, generator=gen, device=device, dtype=torch.float32) * INIT_STD
        q[i : i + n], s[i : i + n] = quantize_blockwise(w)
    return q.reshape(*lead, R, C), s.reshape(*lead, R // BLOCK, C // BLOCK)


def random_rank_model(cfg: ModelConfig, tp: int, rank: int, device, seed: int = 0, cp: bool = False) -> Dict:
    """Random-init shards of the exact geometry generated straight on ``device``.

    Tensors that are replicated across ranks (norms, router, embedding, conv taps of shared
    kv heads) come from a generator seeded by ``seed`` only, rank-local slices from
    ``(seed, rank)``: the model is the concatenation of the shards.  Used by the benchmarks,
    where a global 400 GB tensor set can never exist on one host.  With ``cp`` the ranks that share
    a kv head draw the query rows of their whole group from a group-seeded generator, so every rank
    can also hold the context-parallel front (all the group's query heads) and it agrees with the
    per-rank fronts of its neighbours.
    """
    spec = ShardSpec(cfg, tp, rank)
    shared = torch.Generator(device=device).manual_seed(seed)
    local = torch.Generator(device=device).manual_seed(seed * 1000003 + 17 + rank)
    H, bf = cfg.hidden, torch.bfloat16
    rn = lambda g, *shape: torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * INIT_STD
    layers = []
    for layer in range(cfg.n_layers):
        in_ln, post_ln = 1.0 + rn(shared, H), 1.0 + rn(shared, H)
        if cfg.layer_types[layer] == "linear":
            nv = spec.gdn_v
            fw, fs = _rand_fp8(local, (spec.gdn_front_rows, H), device)
            ow, os_ = _rand_fp8(local, (H, spec.gdn_local), device)
            mix = {
                "kind": "linear", "in_ln": in_ln, "front_w": fw, "front_s": fs,
                "ba_w": rn(local, 2 * nv, H).to(bf),
                "conv_w": (rn(local, spec.gdn_qkv_rows, cfg.conv_kernel) * 10.0).to(bf).float(),
                "a_log": rn(local, nv), "dt_bias": rn(local, nv),
                "gnorm_w": (1.0 + rn(shared, cfg.gdn_dim)).to(bf).float(),
                "out_w": ow, "out_s": os_,
            }
        else:
            # the kv rows must agree inside the group of ranks sharing the kv head
            kvgen = torch.Generator(device=device).manual_seed(seed * 7919 + 31 * layer + spec.kv_head0)
            hd = cfg.head_dim
            cp_front = None
            if cp and spec.cp_size > 1:
                ggen = torch.Generator(device=device).manual_seed(seed * 104729 + 97 * layer + 13 * spec.kv_head0 + 5)
                n_all, hb = spec.q_heads * spec.cp_size, hd // BLOCK
                gw, gs = _rand_fp8(ggen, (n_all * 2 * hd, H), device)          # [(q | gate) per head] of the whole group
                gw8 = gw.view(torch.uint8)
                own = slice(spec.cp_rank * spec.q_heads * 2 * hd, (spec.cp_rank + 1) * spec.q_heads * 2 * hd)
                owns = slice(spec.cp_rank * spec.q_heads * 2 * hb, (spec.cp_rank + 1) * spec.q_heads * 2 * hb)
                qw, qs = gw8[own].contiguous().view(FP8), gs[owns].contiguous()
                heads = range(n_all)
                mine = range(spec.cp_rank * spec.q_heads, (spec.cp_rank + 1) * spec.q_heads)
                cp_front = (
                    [gw8[h * 2 * hd : h * 2 * hd + hd] for h in heads] + [gw8[h * 2 * hd + hd : (h + 1) * 2 * hd] for h in mine],
                    [gs[h * 2 * hb : h * 2 * hb + hb] for h in heads] + [gs[h * 2 * hb + hb : (h + 1) * 2 * hb] for h in mine],
                )
            else:
                qw, qs = _rand_fp8(local, (spec.q_heads * 2 * hd, H), device)
            kw, ks = _rand_fp8(kvgen, (2 * spec.kv_heads * hd, H), device)
            ow, os_ = _rand_fp8(local, (H, spec.attn_local), device)
            mix = {
                "kind": "full", "in_ln": in_ln,
                "front_w": torch.cat([qw.view(torch.uint8), kw.view(torch.uint8)], 0).view(FP8),
                "front_s": torch.cat([qs, ks], 0),
                "qn": 1.0 + rn(shared, hd), "kn": 1.0 + rn(shared, hd),
                "out_w": ow, "out_s": os_,
            }
        E, Il = cfg.n_experts, spec.inter
        w13, w13s = _rand_fp8(local, (E + 1, 2 * Il, H), device)
        w2, w2s = _rand_fp8(local, (E + 1, H, Il), device)
        moe = {
            "post_ln": post_ln, "router_w": rn(shared, E + 1, H).to(bf),
            "w13": w13, "w13_s": w13s, "w2": w2, "w2_s": w2s,
        }
        entry = {"mixer": mix, "moe": moe}
        if cfg.layer_types[layer] != "linear" and cp_front is not None:
            entry["mixer_cp"] = {
                "front_w": torch.cat(cp_front[0] + [kw.view(torch.uint8)], 0).contiguous().view(FP8),
                "front_s": torch.cat(cp_front[1] + [ks], 0).contiguous(),
            }
        layers.append(entry)
    head = {
        "embed": rn(shared, cfg.vocab, H).to(bf),
        "final_ln": 1.0 + rn(shared, H),
        "lm_head": rn(local, spec.vocab, H).to(bf),
    }
    return {"spec": spec, "layers": layers, "head": head}
