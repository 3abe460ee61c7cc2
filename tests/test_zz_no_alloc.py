"""The allocation-free router entry point (csrc/no_alloc.h) called through its exported C symbol.

Some callers of the library cannot create device memory when they need a routing decision (a
plugin handed only a stream and pointers, a thread inside someone else's stream capture, a path
where cudaMalloc's device synchronisation is not acceptable).  For them the router's scratch lives
in a static device array inside the library.  The test checks that entry point against the regular
one, which takes caller-allocated scratch, on two calls in a row (the second call finds the array
holding the first call's contents).  It runs last so that a failure here cannot hide another test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _router_inputs(M, H, E, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(M, H, generator=g, device="cuda") * 2).to(torch.bfloat16)
    ln = 1.0 + 0.02 * torch.randn(H, generator=g, device="cuda")
    rows_pad = (E + 1 + 15) // 16 * 16
    w = torch.zeros(rows_pad, H, dtype=torch.bfloat16, device="cuda")
    w[: E + 1] = (torch.randn(E + 1, H, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    return x, ln, w, rows_pad


# one row, the two-row and four-row instantiations, and eight rows of the full geometry: the array used up to its last float
@pytest.mark.parametrize("M,H,E,topk", [(1, 4096, 512, 10), (4, 1024, 16, 4), (2, 1024, 16, 4), (8, 4096, 512, 10)])
def test_noalloc_router_matches_regular_entry_point(M, H, E, topk):
    from nexrt_b200.ops import lib as L

    lib = L.load()
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = lib.nexrt_moe_router_noalloc
    fn.argtypes = [vp] * 5 + [ci] * 5 + [cf, vp]
    fn.restype = ci
    S = topk + 1
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        x, ln, w, rows_pad = _router_inputs(M, H, E, seed=10 + call)
        # regular entry point with caller-owned scratch
        logits = torch.zeros(M, E + 1, device="cuda")
        partial = torch.zeros(4, M, rows_pad, device="cuda")
        ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
        ids_ref = torch.zeros(M, S, dtype=torch.int32, device="cuda")
        wts_ref = torch.zeros(M, S, device="cuda")
        L.check(lib.nexrt_moe_router(x.data_ptr(), ln.data_ptr(), w.data_ptr(), logits.data_ptr(), ids_ref.data_ptr(), wts_ref.data_ptr(),
                                     ticket.data_ptr(), partial.data_ptr(), rows_pad, H, E, topk, M, 1e-6, 148, None, stream), "router")
        ids = torch.full((M, S), -7, dtype=torch.int32, device="cuda")
        wts = torch.zeros(M, S, device="cuda")
        L.check(fn(x.data_ptr(), ln.data_ptr(), w.data_ptr(), ids.data_ptr(), wts.data_ptr(), rows_pad, H, E, topk, M, 1e-6, stream), "router_noalloc")
        torch.cuda.synchronize()
        assert torch.equal(ids.cpu(), ids_ref.cpu()), (call, ids, ids_ref)
        assert torch.allclose(wts.cpu(), wts_ref.cpu(), rtol=1e-5, atol=1e-6)
        # and against plain PyTorch fp32
        xf = x.float()
        xn = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * ln
        lg = xn @ w[: E + 1].float().T
        top = lg[:, :E].topk(topk, dim=-1)
        assert torch.equal(torch.sort(top.indices, -1).values.cpu(), torch.sort(ids[:, :topk].long(), -1).values.cpu())
        assert torch.allclose(torch.softmax(top.values, -1).cpu(), wts[:, :topk].cpu(), rtol=2e-2, atol=2e-3)
        assert torch.allclose(torch.sigmoid(lg[:, E]).cpu(), wts[:, topk].cpu(), rtol=2e-2, atol=2e-3)


def test_noalloc_router_rejects_oversize():
    from nexrt_b200.ops import lib as L

    lib = L.load()
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = lib.nexrt_moe_router_noalloc
    fn.argtypes = [vp] * 5 + [ci] * 5 + [cf, vp]
    fn.restype = ci
    assert fn(None, None, None, None, None, 528, 4096, 512, 10, 9, 1e-6, None) != 0     # too many rows
    assert fn(None, None, None, None, None, 544, 4096, 512, 10, 1, 1e-6, None) != 0     # too many expert rows
    assert fn(None, None, None, None, None, 528, 8192, 512, 10, 1, 1e-6, None) != 0     # hidden too wide
