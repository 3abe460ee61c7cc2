"""fp32 oracle of the DFlash block draft on the CPU.

The reference has no oracle of its draft stack; its tests pin the kernels one by one
(``nex_n2_5_pro/tests/test_dflash_*``) and the stream end to end.  This one restates the whole draft
(``nex_n2_5_pro/dflash/block.py:152-692``) in plain PyTorch so that the proposals ``ids[1..7]`` and the draft's K/V
caches can be asserted directly:

    context row of a committed position p   c_p = bf16(fc @ cat(taps of p));  per layer k, v = Wk, Wv @ rms(c_p, hidden_norm);
                                            K[p] = bf16(rope(rms(k, k_norm), p)),  V[p] = bf16(v)
    draft block at base position C          rows = [embed(pending), embed(mask) x 7];  per layer: q, k, v from rms(x, in_ln);
                                            block K/V stored at C + m like the context rows;  every row attends every key in
                                            [lo, C + 8) (lo = C + 8 - window on sliding layers), no output gate;  o-proj,
                                            SwiGLU MLP, both with a bf16 residual;  final norm, shared LM head, argmax per row

Rounding contract: weights and residual rows bf16, K/V bf16, everything else fp32.
"""

from __future__ import annotations

from typing import Dict, List, Tuple

import torch
import torch.nn.functional as F

from ..models.reference import partial_rope, rms_norm
from .config import DFlashConfig


class RefDFlashDraft:
    def __init__(self, dc: DFlashConfig, ckpt: Dict[str, torch.Tensor], embed: torch.Tensor, lm_head: torch.Tensor):
        self.dc = dc
        f = lambda t: t.to(torch.bfloat16).float()
        g1 = lambda t: 1.0 + t.float()
        self.embed, self.lm_head = embed.float(), lm_head.float()
        self.fc = f(ckpt["fc.weight"])
        self.hidden_ln, self.final_ln = g1(ckpt["hidden_norm.weight"]), g1(ckpt["norm.weight"])
        self.layers = []
        for l in range(dc.n_layers):
            p = f"layers.{l}."
            self.layers.append({
                "in_ln": g1(ckpt[p + "input_layernorm.weight"]), "post_ln": g1(ckpt[p + "post_attention_layernorm.weight"]),
                "q": f(ckpt[p + "self_attn.q_proj.weight"]), "k": f(ckpt[p + "self_attn.k_proj.weight"]), "v": f(ckpt[p + "self_attn.v_proj.weight"]),
                "o": f(ckpt[p + "self_attn.o_proj.weight"]), "qn": g1(ckpt[p + "self_attn.q_norm.weight"]), "kn": g1(ckpt[p + "self_attn.k_norm.weight"]),
                "gate": f(ckpt[p + "mlp.gate_proj.weight"]), "up": f(ckpt[p + "mlp.up_proj.weight"]), "down": f(ckpt[p + "mlp.down_proj.weight"]),
                "window": dc.sliding_window if dc.layer_types[l] == "sliding" else 0,
            })
        self.reset()

    def reset(self) -> None:
        # per layer: position -> (K [kv, hd], V [kv, hd]); a later write to a position replaces the earlier one
        self.k: List[Dict[int, torch.Tensor]] = [dict() for _ in self.layers]
        self.v: List[Dict[int, torch.Tensor]] = [dict() for _ in self.layers]

    def _store(self, layer: int, pos: int, k: torch.Tensor, v: torch.Tensor) -> None:
        dc, w = self.dc, self.layers[layer]
        k = partial_rope(rms_norm(k.reshape(dc.n_kv_heads, dc.head_dim), w["kn"], dc.rms_eps), pos, dc.rotary_dim, dc.rope_theta)
        self.k[layer][pos] = k.to(torch.bfloat16).float()
        self.v[layer][pos] = v.reshape(dc.n_kv_heads, dc.head_dim).to(torch.bfloat16).float()

    @torch.inference_mode()
    def context(self, pos: int, taps: torch.Tensor) -> None:
        """Committed position ``pos`` with its target features ``taps`` (concatenated bf16 rows of the tapped layers)."""
        c = (self.fc @ taps.float()).to(torch.bfloat16)
        cn = rms_norm(c, self.hidden_ln, self.dc.rms_eps)
        for l, w in enumerate(self.layers):
            self._store(l, pos, w["k"] @ cn, w["v"] @ cn)

    @torch.inference_mode()
    def draft(self, pending: int, base: int) -> Tuple[List[int], torch.Tensor]:
        """The eight-row block at base position ``base``: returns (argmax of every row, logits [8, vocab]).  Rows 1..7 are
        the proposals; the block's own K/V rows stay in the caches until the next context rows replace them."""
        dc = self.dc
        rows = 8
        x = torch.stack([self.embed[pending]] + [self.embed[dc.mask_token_id]] * (rows - 1)).to(torch.bfloat16)
        rep = dc.n_q_heads // dc.n_kv_heads
        for l, w in enumerate(self.layers):
            xn = torch.stack([rms_norm(x[m], w["in_ln"], dc.rms_eps) for m in range(rows)])
            q, k, v = xn @ w["q"].T, xn @ w["k"].T, xn @ w["v"].T
            for m in range(rows):
                self._store(l, base + m, k[m], v[m])
            hi = base + rows
            lo = max(0, hi - w["window"]) if w["window"] > 0 else 0
            keys = [p for p in range(lo, hi)]
            missing = [p for p in keys if p not in self.k[l]]
            if missing:
                raise KeyError(f"draft layer {l}: no context row for positions {missing[:4]}...")
            K = torch.stack([self.k[l][p] for p in keys], 1).repeat_interleave(rep, 0)      # [q heads, S, hd]
            V = torch.stack([self.v[l][p] for p in keys], 1).repeat_interleave(rep, 0)
            out = []
            for m in range(rows):
                qm = partial_rope(rms_norm(q[m].reshape(dc.n_q_heads, dc.head_dim), w["qn"], dc.rms_eps), base + m, dc.rotary_dim, dc.rope_theta)
                scores = torch.einsum("hd,hsd->hs", qm, K) * dc.head_dim ** -0.5
                out.append(torch.einsum("hs,hsd->hd", torch.softmax(scores, -1), V).reshape(-1))
            x = (x.float() + torch.stack(out) @ w["o"].T).to(torch.bfloat16)
            xn = torch.stack([rms_norm(x[m], w["post_ln"], dc.rms_eps) for m in range(rows)])
            x = (x.float() + (F.silu(xn @ w["gate"].T) * (xn @ w["up"].T)) @ w["down"].T).to(torch.bfloat16)
        logits = torch.stack([self.lm_head @ rms_norm(x[m], self.final_ln, dc.rms_eps) for m in range(rows)])
        return [int(t) for t in logits.argmax(-1)], logits

    def kv(self, layer: int, upto: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """K, V ``[kv heads, upto, hd]`` of positions ``0 .. upto - 1``."""
        return (torch.stack([self.k[layer][p] for p in range(upto)], 1), torch.stack([self.v[layer][p] for p in range(upto)], 1))
