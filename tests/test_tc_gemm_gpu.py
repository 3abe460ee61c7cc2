"""tcgen05 GEMM against fp32 PyTorch: block-scaled FP8 (exact dequantised operands), BF16, ragged
token / row counts, accumulate mode, and the CUDA activation quantiser against the host one."""

import pytest
import torch

from nexrt_b200.ops.tc_gemm import act_quant, bf16_gemm, fp8_gemm
from nexrt_b200.quant import act_quant as act_quant_ref
from nexrt_b200.quant import dequantize_blockwise, quantize_blockwise

pytestmark = pytest.mark.gpu


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-20))


def _deq_act(xq, sx):
    T, K = xq.shape
    return (xq.float().reshape(T, K // 128, 128) * sx[..., None]).reshape(T, K)


@pytest.mark.parametrize("T,R,K", [(8, 256, 512), (16, 128, 128), (33, 384, 1024), (64, 2560, 4096), (128, 1024, 4096), (5, 200, 256)])
def test_fp8_block_scaled_gemm(T, R, K):
    g = torch.Generator(device="cuda").manual_seed(T * 1000 + R)
    w = torch.randn(R, K, device="cuda", generator=g) * 0.05
    pad = (128 - R % 128) % 128
    wq_full, sw = quantize_blockwise(torch.cat([w, torch.zeros(pad, K, device="cuda")]) if pad else w)
    wq = wq_full[:R].contiguous()
    x = (torch.randn(T, K, device="cuda", generator=g) * 2).to(torch.bfloat16)
    xq, sx = act_quant(x)
    want = _deq_act(xq, sx).double() @ dequantize_blockwise(wq_full, sw)[:R].double().T
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = fp8_gemm(wq, sw, xq, sx, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert got.shape == (T, R) and rel(got, want) < 1e-5
    # and it is a faithful product of the unquantised operands to FP8 accuracy
    assert rel(got, x.double() @ w.double().T) < 0.06
    got_bf = fp8_gemm(wq, sw, xq, sx, out_dtype=torch.bfloat16)
    assert rel(got_bf, want) < 5e-3
    acc = want.float().clone()
    fp8_gemm(wq, sw, xq, sx, out=acc, accumulate=True)
    assert rel(acc, 2 * want) < 1e-5


@pytest.mark.parametrize("T,R,K", [(8, 128, 64), (16, 256, 512), (40, 300, 1024), (64, 4096, 4096)])
def test_bf16_gemm(T, R, K):
    g = torch.Generator(device="cuda").manual_seed(R)
    w = (torch.randn(R, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    x = torch.randn(T, K, device="cuda", generator=g).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = bf16_gemm(w, x, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and rel(got, x.double() @ w.double().T) < 1e-5
    # strided activations (a column window of a wider buffer)
    wide = torch.randn(T, 2 * K, device="cuda", generator=g).to(torch.bfloat16)
    assert rel(bf16_gemm(w, wide[:, K:]), wide[:, K:].double() @ w.double().T) < 1e-5


def test_act_quant_matches_host_quantiser_and_fuses_rmsnorm():
    g = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn(19, 1024, device="cuda", generator=g) * 3).to(torch.bfloat16)
    xq, sx = act_quant(x)
    q_ref, s_ref = act_quant_ref(x.cpu())
    assert torch.allclose(sx.cpu(), s_ref, rtol=1e-6) and rel(_deq_act(xq, sx).cpu(), _deq_act(q_ref, s_ref)) < 4e-3
    gamma = 1 + 0.1 * torch.randn(1024, device="cuda", generator=g)
    xn = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * gamma
    xq2, sx2 = act_quant(x, gamma)
    assert rel(_deq_act(xq2, sx2), xn) < 0.04
    xq3, sx3 = act_quant(xn)            # fp32 input path
    assert rel(_deq_act(xq3, sx3), xn) < 0.04
