"""tcgen05 expert kernels (gate/up with one pass per distinct expert, down projection + all-reduce epilogue +
residual) against an fp32 evaluation of the same block-scaled FP8 experts."""

import ctypes

import pytest
import torch

from nexrt_b200.ops.lib import check, load, ptr
from nexrt_b200.parallel.channel import LLChannel
from nexrt_b200.quant import dequantize_blockwise, quantize_blockwise

pytestmark = pytest.mark.gpu


def rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-20))


@pytest.mark.parametrize("ksplit", [1, 2])
@pytest.mark.parametrize("H,I,E,S,M", [(1024, 256, 16, 5, 8), (4096, 128, 48, 11, 8), (4096, 128, 48, 11, 4), (1024, 128, 8, 3, 2)])
def test_expert_kernels_match_fp32(H, I, E, S, M, ksplit):
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(H + I + M)
    w13 = torch.randn(E + 1, 2 * I, H, device=dev, generator=g) * 0.03
    w2 = torch.randn(E + 1, H, I, device=dev, generator=g) * 0.03
    w13q, w13s = quantize_blockwise(w13)
    w2q, w2s = quantize_blockwise(w2)
    x = (torch.randn(M, H, device=dev, generator=g) * 1.5).to(torch.bfloat16)
    gamma = 1 + 0.1 * torch.randn(H, device=dev, generator=g)
    # routing: distinct experts per row, overlapping between rows, shared expert (index E) last
    ids = torch.stack([torch.cat([torch.randperm(E, device=dev, generator=g)[: S - 1], torch.tensor([E], device=dev)]) for _ in range(M)]).to(torch.int32)
    wts = torch.rand(M, S, device=dev, generator=g) * 0.3 + 0.05
    lib = load()
    st = torch.cuda.current_stream().cuda_stream
    gu_planes = torch.zeros(ksplit, M, S, 2 * I, device=dev)
    planes1 = torch.zeros(3 * 8, H, dtype=torch.uint8, device=dev)
    planes2 = torch.zeros(3 * 8, S * I, dtype=torch.uint8, device=dev)
    descale = torch.zeros(8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    check(lib.nexrt_tc_moe_l1(ptr(x), ptr(gamma), ptr(w13q), ptr(w13s), ptr(ids), ptr(gu_planes), ptr(planes1), H, I, S, M, E + 1, ksplit, 1e-6, 0, ptr(status), st), "l1")
    torch.cuda.synchronize()
    gu = gu_planes.sum(0)
    xn = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * gamma
    w13d = dequantize_blockwise(w13q.reshape(-1, H), w13s.reshape(-1, H // 128)).reshape(E + 1, 2 * I, H)
    want_gu = torch.einsum("msrh,mh->msr", w13d[ids.long()], xn)
    assert int(status.item()) == 0 and rel(gu, want_gu) < 2e-3, rel(gu, want_gu)
    # down projection + (single-rank) all-reduce + residual
    ch = LLChannel(dev, 1, 0, 8 * H)
    xres = x.clone()
    check(lib.nexrt_tc_moe_l2_allreduce(ptr(gu_planes), ptr(ids), ptr(wts), ptr(w2q), ptr(w2s), ptr(xres), ptr(planes2), ptr(descale), H, I, S, M, E + 1, ksplit,
                                        ch.ref, 0, ptr(status), st), "l2")
    torch.cuda.synchronize()
    h = torch.nn.functional.silu(gu[..., :I]) * gu[..., I:] * wts[..., None]
    w2d = dequantize_blockwise(w2q.reshape(-1, I), w2s.reshape(-1, I // 128)).reshape(E + 1, H, I)
    y = torch.einsum("mshi,msi->mh", w2d[ids.long()], h)
    want = (x.float() + y).to(torch.bfloat16)
    assert int(status.item()) == 0
    assert rel(xres.float() - x.float(), y) < 6e-2, rel(xres.float() - x.float(), y)       # bf16 rounding of x + y dominates
    assert (xres.float() - want.float()).abs().max() <= 2 * torch.finfo(torch.bfloat16).eps * want.float().abs().max()


@pytest.mark.parametrize("mode,K,M", [(0, 1024, 8), (1, 1024, 4), (1, 512, 8), (0, 2048, 5)])
def test_wide_out_projection_matches_the_fused_kernel(mode, K, M):
    """Staging + tcgen05 GEMM with the all-reduce epilogue against the fused mma.sync out-projection kernel."""
    dev = torch.device("cuda", 0)
    H = 1024
    g = torch.Generator(device=dev).manual_seed(K + M + mode)
    wq, ws = quantize_blockwise(torch.randn(H, K, device=dev, generator=g) * 0.03)
    inp = torch.randn(8, K, device=dev, generator=g)
    z = torch.randn(8, K, device=dev, generator=g)
    gnorm = 1 + 0.1 * torch.randn(128, device=dev, generator=g)
    x0 = torch.randn(8, H, device=dev, generator=g).to(torch.bfloat16)
    lib, st = load(), torch.cuda.current_stream().cuda_stream
    ch = LLChannel(dev, 1, 0, 8 * H)
    x_ref = x0.clone()
    check(lib.nexrt_oproj_allreduce(ptr(inp), ptr(z), ptr(gnorm), ptr(wq), ptr(ws), ptr(x_ref), H, K, M, mode, 1e-6, 128, ch.ref, 0, None, 0, 148, st), "fused")
    x_new = x0.clone()
    planes = torch.zeros(24, K, dtype=torch.uint8, device=dev)
    descale = torch.zeros(8, device=dev)
    zero = torch.zeros(8, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    check(lib.nexrt_oproj_stage_split(ptr(inp), ptr(z), ptr(gnorm), ptr(planes), ptr(descale), K, M, mode, 1e-6, 128, None, 0, st), "stage")
    check(lib.nexrt_tc_oproj_allreduce(ptr(planes), ptr(descale), ptr(wq), ptr(ws), ptr(x_new), ptr(zero), H, K, M, 0, ch.ref, 1, ptr(status), st), "wide")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(x_new[M:], x0[M:])                                  # rows beyond M untouched
    d_ref, d_new = x_ref[:M].float() - x0[:M].float(), x_new[:M].float() - x0[:M].float()
    assert rel(d_new, d_ref) < 3e-2                                       # both are bf16-rounded sums of the same fp32 result
    assert (x_new[:M].float() - x_ref[:M].float()).abs().max() <= 2 * torch.finfo(torch.bfloat16).eps * x_ref[:M].float().abs().max()
