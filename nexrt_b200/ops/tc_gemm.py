"""Python face of the tcgen05 GEMM (``csrc/tc_gemm.cu``): block-scaled FP8 and BF16 products of a token
block with a weight matrix, used wherever more than a handful of rows meet the same weights (prefill
chunks, wide verify).  Shapes follow the checkpoint: weights ``[R, K]`` row-major (FP8 with one fp32
scale per 128 x 128 block, reference ``nex_n2_5_pro/weights.py:27-31``), activations ``[T, K]``.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..quant import FP8
from .lib import check, load as lib, ptr


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def act_quant(x: torch.Tensor, gamma: Optional[torch.Tensor] = None, eps: float = 1e-6, terms: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [T, K]`` (bf16 or fp32, last dim contiguous) -> (e4m3 ``[terms * T, K]``, fp32 scales ``[terms * T, K/128]``);
    with ``gamma`` (the full RMSNorm multiplier, fp32 ``[K]``) the rows are normalised first.  ``terms`` > 1 writes the
    step kernels' exact split as further row blocks: block ``p`` holds the residual of the blocks before it at a 16 times
    finer scale, so ``sum_p fp8_gemm(...)[p * T : (p + 1) * T]`` multiplies by ``x`` to 2^-8 (two terms) or 2^-12 (three)."""
    if x.dim() != 2 or x.stride(1) != 1 or x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("act_quant expects a 2-D bf16/fp32 tensor with contiguous rows")
    if terms not in (1, 2, 3):
        raise ValueError("act_quant: terms must be 1, 2 or 3")
    T, K = x.shape
    xq = torch.empty(terms * T, K, dtype=FP8, device=x.device)
    sx = torch.empty(terms * T, K // 128, dtype=torch.float32, device=x.device)
    check(lib().nexrt_act_quant(ptr(x), int(x.dtype == torch.float32), x.stride(0), ptr(gamma), eps, ptr(xq), ptr(sx), T, K, terms, _stream()), "act_quant")
    return xq, sx


def fp8_gemm(wq: torch.Tensor, sw: torch.Tensor, xq: torch.Tensor, sx: torch.Tensor, out: Optional[torch.Tensor] = None,
             out_dtype: torch.dtype = torch.float32, accumulate: bool = False, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``Y[T, R] = dequant(xq, sx) @ dequant(wq, sw).T`` on the tensor cores."""
    R, K = wq.shape
    T = xq.shape[0]
    if xq.shape[1] != K or not xq.is_contiguous() or wq.stride(1) != 1:
        raise ValueError("fp8_gemm: operand shapes / strides")
    if tuple(sw.shape) != ((R + 127) // 128, K // 128) or tuple(sx.shape) != (T, K // 128) or not (sw.is_contiguous() and sx.is_contiguous()):
        raise ValueError("fp8_gemm: scale shapes")
    if out is None:
        out = torch.empty(T, R, dtype=out_dtype, device=wq.device)
    mode = 2 if accumulate else (0 if out.dtype == torch.float32 else 1)
    if accumulate and out.dtype != torch.float32:
        raise ValueError("accumulate needs an fp32 output")
    check(lib().nexrt_tc_gemm_fp8(ptr(wq), ptr(sw), wq.stride(0), ptr(xq), ptr(sx), ptr(out), T, R, K, out.stride(0), mode, ptr(status), _stream()), "tc_gemm_fp8")
    return out


def bf16_gemm(w: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.float32,
              accumulate: bool = False, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``Y[T, R] = x @ w.T`` with bf16 operands and fp32 accumulation on the tensor cores."""
    R, K = w.shape
    T = x.shape[0]
    if x.shape[1] != K or w.stride(1) != 1 or x.stride(1) != 1 or w.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
        raise ValueError("bf16_gemm: operand shapes / dtypes")
    if out is None:
        out = torch.empty(T, R, dtype=out_dtype, device=w.device)
    mode = 2 if accumulate else (0 if out.dtype == torch.float32 else 1)
    check(lib().nexrt_tc_gemm_bf16(ptr(w), w.stride(0), ptr(x), x.stride(0), ptr(out), T, R, K, out.stride(0), mode, ptr(status), _stream()), "tc_gemm_bf16")
    return out


def fp8_gemm_split(wq: torch.Tensor, sw: torch.Tensor, xq: torch.Tensor, sx: torch.Tensor, out: torch.Tensor, ksplit: int = 1,
                   group_k: int = 0, group_rows: int = 0, used: Optional[torch.Tensor] = None, used_rows: int = 0,
                   status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The block-scaled FP8 product with K split over ``ksplit`` CTAs per tile: ``out [ksplit, T, R]`` fp32 partial
    planes (add them in plane order).  With ``group_rows`` the weight is a stack of ``K / group_k`` matrices
    ``[group_rows, group_k]`` (the experts' down projections, ``w2 [E+1, H, I]`` viewed as ``[(E+1) * H, I]``) whose
    K extents are concatenated: ``out[t, r] = sum_g x[t, g*group_k:(g+1)*group_k] . w[g, r, :]``.  ``used`` (int32, one
    entry per group) leaves out what nothing is routed to: with a stack, the K blocks of unused groups; with a plain
    matrix whose rows come in groups of ``used_rows``, the row tiles of unused groups (their output is not written)."""
    T, K = xq.shape
    R = group_rows if group_rows else wq.shape[0]
    if out.dtype != torch.float32 or out.numel() < ksplit * T * R or not (xq.is_contiguous() and sx.is_contiguous() and sw.is_contiguous()):
        raise ValueError("fp8_gemm_split: output / operand layout")
    check(lib().nexrt_tc_gemm_fp8_ex(ptr(wq), ptr(sw), wq.stride(0), ptr(xq), ptr(sx), ptr(out), T, R, K, R, ksplit, group_k, group_rows, ptr(used), used_rows, ptr(status), _stream()),
          "tc_gemm_fp8_ex")
    return out


def bf16_gemm_split(w: torch.Tensor, x: torch.Tensor, out: torch.Tensor, ksplit: int, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The bf16 product with K split over ``ksplit`` CTAs per tile: ``out [ksplit, T, R]`` fp32 partial planes."""
    R, K = w.shape
    T = x.shape[0]
    if x.shape[1] != K or w.stride(1) != 1 or x.stride(1) != 1 or out.dtype != torch.float32 or out.numel() < ksplit * T * R or not out.is_contiguous():
        raise ValueError("bf16_gemm_split: operand / output layout")
    check(lib().nexrt_tc_gemm_bf16_ex(ptr(w), w.stride(0), ptr(x), x.stride(0), ptr(out), T, R, K, R, ksplit, ptr(status), _stream()), "tc_gemm_bf16_ex")
    return out
