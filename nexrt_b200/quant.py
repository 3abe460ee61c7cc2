"""FP8 e4m3 quantisation with 128x128 block scales (weights) and 1x128 group scales (activations).

Weight recipe follows the reference's requantiser ``nex_n2_5_pro/gdn.py:71-80``:
``scale = amax(block) / 448`` clamped below at 1e-12, ``q = clamp(w / scale, +-448)`` rounded
to e4m3.  The stored scale is the dequantisation multiplier (the checkpoint's
``weight_scale_inv``; ``nex_n2_5_pro/weights.py:27-31`` accepts both names).  Activation recipe
follows ``nex_n2_5_pro/attn.py:87-94`` (dynamic per row, per 128 elements).
"""

from __future__ import annotations

import torch

from .config import BLOCK

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


def _ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def quantize_blockwise(w: torch.Tensor):
    """``w [..., R, C]`` float -> (``q`` fp8 same shape, ``scale [..., ceil(R/128), ceil(C/128)]`` fp32)."""
    *lead, R, C = w.shape
    RB, CB = _ceil_div(R, BLOCK), _ceil_div(C, BLOCK)
    wf = w.float()
    if R % BLOCK or C % BLOCK:
        pad = torch.zeros(*lead, RB * BLOCK, CB * BLOCK, dtype=torch.float32, device=w.device)
        pad[..., :R, :C] = wf
        wf = pad
    wb = wf.reshape(*lead, RB, BLOCK, CB, BLOCK)
    scale = (wb.abs().amax(dim=(-3, -1)) / FP8_MAX).clamp_min(1e-12)
    q = (wb / scale[..., :, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    q = q.reshape(*lead, RB * BLOCK, CB * BLOCK)[..., :R, :C].contiguous()
    return q, scale.contiguous()


def dequantize_blockwise(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`quantize_blockwise` in fp32."""
    *_, R, C = q.shape
    s = scale.float().repeat_interleave(BLOCK, -2)[..., :R, :].repeat_interleave(BLOCK, -1)[..., :C]
    return q.float() * s


def fold_requant(q: torch.Tensor, scale: torch.Tensor, gamma: torch.Tensor):
    """Fold a per-input-column multiplier into a block-scaled weight with fresh scales
    (reference ``_fold_requant_2d``, gdn.py:71-80).  ``gamma [C]`` fp32."""
    w = dequantize_blockwise(q, scale) * gamma.float().view(*([1] * (q.dim() - 1)), -1)
    return quantize_blockwise(w)


def act_quant(x: torch.Tensor):
    """Per-row, per-128-element dynamic FP8 activation quantisation.

    ``x [rows, K]`` -> (``q`` fp8 ``[rows, K]``, ``scale [rows, K/128]`` fp32) with
    ``scale = max(amax, 1e-10) / 448``.
    """
    rows, K = x.shape
    if K % BLOCK:
        raise ValueError("activation width must be a multiple of 128")
    blocks = x.float().reshape(rows, K // BLOCK, BLOCK)
    scale = blocks.abs().amax(-1, keepdim=True).clamp_min(1e-10) / FP8_MAX
    q = (blocks / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q.reshape(rows, K), scale.reshape(rows, K // BLOCK).contiguous()


def act_quant_terms(x: torch.Tensor, terms: int = 3):
    """The wide prefill path's activation split, in the layout and the arithmetic of its quantiser kernels
    (``csrc/prefill.cu: quant_block4``, ``csrc/tc_gemm.cu: act_quant_kernel``).

    ``x [rows, K]`` -> (``q`` fp8 ``[terms * rows, K]``, ``scale [terms * rows, K/128]``): row block 0 is
    ``e4m3(x / s)`` with ``s = max(amax, 1e-12) / 448`` per row and 128 columns; row block ``p`` is the e4m3 rounding of what
    the blocks before it left over, at the scale ``s / 16^p`` (the residual is multiplied by 16 before it is rounded, so that
    every term uses e4m3's normal range).  ``sum_p q_p * s_p`` equals ``x`` to 2^-4, 2^-8, 2^-12 of each value for 1, 2, 3
    terms, and a GEMM over all ``terms * rows`` rows followed by the sum of its row blocks multiplies by that sum.
    """
    if terms not in (1, 2, 3):
        raise ValueError("terms must be 1, 2 or 3")
    rows, K = x.shape
    if K % BLOCK:
        raise ValueError("activation width must be a multiple of 128")
    blocks = x.float().reshape(rows, K // BLOCK, BLOCK)
    scale = blocks.abs().amax(-1, keepdim=True).clamp_min(1e-12) / FP8_MAX
    r = blocks * (1.0 / scale)
    qs, ss = [], []
    for p in range(terms):
        q = r.clamp(-FP8_MAX, FP8_MAX).to(FP8)
        qs.append(q.reshape(rows, K))
        ss.append((scale / 16.0 ** p).reshape(rows, K // BLOCK))
        r = (r - q.float()) * 16.0
    return torch.cat(qs), torch.cat(ss).contiguous()


def act_quant_dequant(x: torch.Tensor) -> torch.Tensor:
    q, s = act_quant(x)
    return (q.float().reshape(x.shape[0], -1, BLOCK) * s[..., None]).reshape(x.shape)
