"""fp32 oracles of the MTP path on the CPU: the draft layer itself, and the multi-row sample / prefix-accept / commit
step of the verifier.

Counterpart of the reference's CPU oracle ``nex_n2_5_pro/mtp/sampling_ref.py:30-143`` (4-row sample + prefix accept +
commit) extended by what it has no oracle for, the draft layer: one gated-attention + MoE layer of the target's geometry
fed with ``fc(cat[norm_e(emb(token p+1)) | norm_h(norm_f(hidden p))])`` (``nex_n2_5_pro/mtp/block.py:497-576``,
``kernels/mtp/nex_n2_5_pro_mtp_preprocess_ctypes.cu:68-127``).  Rounding contract as in ``models/reference.py``: the
residual rows and the KV cache are bf16, everything else fp32; ``mtp.fc`` is used as quantised at load (FP8 e4m3,
128 x 128 block scales).
"""

from __future__ import annotations

from dataclasses import replace
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..config import ModelConfig
from ..models.reference import RefModel, rms_norm
from ..quant import dequantize_blockwise, quantize_blockwise
from ..sampling import sample_reference
from ..weights import PFX
from .weights import MTP_BASE


class RefMtpDraft:
    """The draft layer, one position at a time along the committed path."""

    def __init__(self, cfg: ModelConfig, target_ckpt: Dict[str, torch.Tensor], mtp_ckpt: Dict[str, torch.Tensor]):
        one = replace(cfg, n_layers=1, layer_types=("full",))
        sub = {
            PFX + "embed_tokens.weight": target_ckpt[PFX + "embed_tokens.weight"],
            PFX + "norm.weight": mtp_ckpt["mtp.norm.weight"],
            "lm_head.weight": target_ckpt["lm_head.weight"],
        }
        sub.update({k.replace(MTP_BASE, PFX + "layers.0."): v for k, v in mtp_ckpt.items() if k.startswith(MTP_BASE)})
        self.cfg = cfg
        self.layer = RefModel(one, sub)
        self.ge = 1.0 + mtp_ckpt["mtp.pre_fc_norm_embedding.weight"].float()
        self.gh = 1.0 + mtp_ckpt["mtp.pre_fc_norm_hidden.weight"].float()
        self.gf = 1.0 + target_ckpt[PFX + "norm.weight"].float()
        self.fc = dequantize_blockwise(*quantize_blockwise(mtp_ckpt["mtp.fc.weight"].float()))

    def reset(self) -> None:
        self.layer.reset()

    @torch.inference_mode()
    def step(self, hidden: torch.Tensor, token: int, pos: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Draft-layer position ``pos``: pairs the hidden row of that position (bf16 residual row of the target, or the
        draft layer's own output in a chained pass) with the token one position later.  Returns ``(logits, hidden_out)``;
        ``argmax(logits)`` is the draft for position ``pos + 2``."""
        c, L = self.cfg, self.layer
        e = L.embed[token]
        cat = torch.cat([rms_norm(e, self.ge, c.rms_eps), rms_norm(rms_norm(hidden.float(), self.gf, c.rms_eps), self.gh, c.rms_eps)])
        x = (self.fc @ cat).to(torch.bfloat16)
        w, st = L.layers[0], L.states[0]
        del st.k[pos:], st.v[pos:]                       # a pass at an earlier position overwrites speculative rows
        x = (x.float() + L._attn(w, st, x, pos)).to(torch.bfloat16)
        x = (x.float() + L._moe(w, x)).to(torch.bfloat16)
        return L.lm_head @ rms_norm(x, L.final_ln, c.rms_eps), x

    def kv(self) -> Tuple[torch.Tensor, torch.Tensor]:
        st = self.layer.states[0]
        return torch.stack(st.k, 1), torch.stack(st.v, 1)


def verify_reference(logits_rows: Sequence[torch.Tensor], ids: Sequence[int], committed_len: int, seed: int, temperature: float, top_p: float,
                     top_k: int, forced_commit: int = 0, upstream_status: int = 0, eos: Optional[int] = None) -> Dict:
    """What the verifier's sampler and commit step must produce for ``M = len(ids)`` rows.

    ``ids[j]`` is the token fed at row ``j`` (``ids[0]`` the pending token, ``ids[1:]`` the drafts) and ``logits_rows[j]``
    the target's logits of that row, i.e. the distribution of the token at position ``committed_len + j + 1``.  Every row is
    sampled with the position-keyed generator of its own position (so a row's token does not depend on how many rows the
    step carried); drafts are accepted while ``target[j] == ids[j + 1]``; ``forced_commit > 0`` overrides the accepted
    count; any upstream failure commits nothing.  Returns the control words the step must leave."""
    M = len(ids)
    target, kept = [], []
    for j in range(M):
        tok, kept_ids, probs = sample_reference(logits_rows[j].tolist(), seed, committed_len + j, temperature, top_p, top_k)
        target.append(tok)
        kept.append((kept_ids, probs))
    if upstream_status:
        return {"status": upstream_status, "commit_count": 0, "accepted": 0, "pending": -1, "emitted": [-1] * 8, "committed_len": committed_len,
                "target": target, "kept": kept}
    accepted = 0
    for j in range(M - 1):
        if accepted == j and target[j] == ids[j + 1]:
            accepted = j + 1
    if forced_commit > 0:
        accepted = min(forced_commit, M) - 1
    commit = accepted + 1
    emitted = [ids[j + 1] if j < accepted else (target[accepted] if j == accepted else -1) for j in range(8)]
    stop = -1
    if eos is not None and eos >= 0:
        for j in range(commit):
            if emitted[j] == eos:
                stop = j
                break
    return {"status": 0, "commit_count": commit, "accepted": accepted, "pending": target[accepted], "emitted": emitted,
            "committed_len": committed_len + commit, "stop_pos": stop, "target": target, "kept": kept}
