"""Worker of tests/test_tp_gpu.py::test_allreduce_ops: the two in-kernel all-reduce protocols as plain operators on 2+ ranks.

1. the packet protocol (``csrc/epilogue.cuh`` through ``nexrt_ll_allreduce_bench``) and the block protocol of the wide
   prefill (``nexrt_planes_allreduce_residual``) give, on every rank, exactly the bits of a rank-ordered fp32 sum;
2. inputs built to cancel (huge values of opposite sign on different ranks plus a small one) give the same bits over 64
   replays of a captured graph while the ranks are skewed against each other by a rank-dependent device sleep before
   every replay (the arrival order of the packets changes, the order of the additions must not; reference:
   tests/test_cp_reduce_determinism.py:59-113);
3. a peer that never calls: the callers' waits run out after the channel's budget, the status word latches
   REDUCE_TIMEOUT, the kernel returns, and after a collective reset the channel works again.
"""

import ctypes
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nexrt_b200.ops import lib as L  # noqa: E402
from nexrt_b200.ops.lib import check, ptr  # noqa: E402
from nexrt_b200.parallel.channel import LLChannel  # noqa: E402
from nexrt_b200.runtime.control import Status  # noqa: E402


def rank_ordered_sum(parts):
    total = torch.zeros_like(parts[0])
    for p in parts:
        total = total + p
    return total


def gather(t):
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return out


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    lib = L.load()
    H = 4096
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ch = LLChannel(dev, world, rank, 8 * H, group=None, budget_ms=5000)
    peer = ch.variant(multicast=False)
    forms = ([("multicast", ch.struct)] if ch.multicast else []) + [("peer-stores", peer)]
    g = torch.Generator(device=dev).manual_seed(100 + rank)

    def packet_allreduce(struct, partial, x, site=0, advance=True):
        check(lib.nexrt_ll_allreduce_bench(ptr(partial), ptr(x), partial.shape[0], H, ctypes.byref(struct), site, None, st), "ll_allreduce_bench")
        if advance:
            check(lib.nexrt_ll_seq_advance(ptr(ch.seq), 1, st), "seq_advance")

    # ---- 1a. packet protocol: bits of the rank-ordered sum, the same on every rank ------------------------------
    for name, struct in forms:
        for M in (1, 4, 8):
            partial = torch.randn(M, H, dtype=torch.float32, device=dev, generator=g)
            x = torch.zeros(M, H, dtype=torch.bfloat16, device=dev)
            packet_allreduce(struct, partial, x)
            torch.cuda.synchronize()
            want = rank_ordered_sum(gather(partial)).to(torch.bfloat16)
            assert torch.equal(x, want), (name, M, float((x.float() - want.float()).abs().max()))
            assert int(ch.status.item()) == 0

    # ---- 1b. block protocol of the wide prefill ------------------------------------------------------------------
    n, ksplit = 16 * H, 3
    blk = LLChannel(dev, world, rank, n, group=None, seq=ch.seq, status=ch.status, budget_ms=5000)
    blk_peer = blk.variant(multicast=False)
    x0 = torch.randn(n, dtype=torch.float32, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).to(torch.bfloat16)
    for name, struct in ([("multicast", blk.struct)] if blk.multicast else []) + [("peer-stores", blk_peer)]:
        y = torch.randn(ksplit, n, dtype=torch.float32, device=dev, generator=g)
        x = x0.clone()
        check(lib.nexrt_planes_allreduce_residual(ptr(x), ptr(y), n, ksplit, ctypes.byref(struct), 0, st), "planes_allreduce_residual")
        check(lib.nexrt_ll_seq_advance(ptr(ch.seq), 1, st), "seq_advance")
        torch.cuda.synchronize()
        own = (y[0] + y[1]) + y[2]
        want = (x0.float() + rank_ordered_sum(gather(own))).to(torch.bfloat16)
        assert torch.equal(x, want), (name, float((x.float() - want.float()).abs().max()))
        same = gather(x)
        assert all(torch.equal(same[0], s) for s in same)
    assert int(ch.status.item()) == 0

    # ---- 2. cancellation pattern under rank skew, 64 graph replays ----------------------------------------------
    M = 8
    partial = torch.randn(M, H, dtype=torch.float32, device=dev, generator=g) * 1e-3
    sign = 1.0 if rank % 2 == 0 else -1.0
    partial += sign * 3.0e7 * (1 + torch.arange(H, device=dev, dtype=torch.float32) % 7)      # cancels pairwise across ranks, not bitwise-commutatively
    x = torch.zeros(M, H, dtype=torch.bfloat16, device=dev)
    struct = forms[0][1]
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        packet_allreduce(struct, partial, x)
        side.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            check(lib.nexrt_ll_allreduce_bench(ptr(partial), ptr(x), M, H, ctypes.byref(struct), 0, None, ctypes.c_void_p(side.cuda_stream)), "ar")
            check(lib.nexrt_ll_seq_advance(ptr(ch.seq), 1, ctypes.c_void_p(side.cuda_stream)), "adv")
    want = rank_ordered_sum(gather(partial)).to(torch.bfloat16)
    seen = None
    for it in range(64):
        x.zero_()
        torch.cuda._sleep(((rank * 7 + it * 3) % world) * 200_000)      # up to a few hundred microseconds of skew, in a different order every replay
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(x, want), it
        if seen is None:
            seen = x.clone()
        assert torch.equal(x, seen)
    same = gather(x)
    assert all(torch.equal(same[0], s) for s in same) and int(ch.status.item()) == 0

    # ---- 3. a peer that stays silent --------------------------------------------------------------------------------
    dist.barrier()
    silent = world - 1
    short = ch.variant(multicast=False, budget_ms=50)
    partial = torch.ones(1, H, dtype=torch.float32, device=dev)
    x = torch.zeros(1, H, dtype=torch.bfloat16, device=dev)
    if rank != silent:
        packet_allreduce(short, partial, x, advance=False)
    torch.cuda.synchronize()
    status = int(ch.status.item())
    assert status == (0 if rank == silent else Status.REDUCE_TIMEOUT), status
    if rank != silent:
        assert float(x.float().max()) <= world - 1         # the silent rank's share is missing, nothing else is
    dist.barrier()
    ch.reset()
    torch.cuda.synchronize()
    dist.barrier()
    packet_allreduce(peer, partial, x)
    torch.cuda.synchronize()
    assert int(ch.status.item()) == 0 and torch.equal(x, torch.full_like(x, float(world)))
    dist.barrier()
    if rank == 0:
        print("AR_WORKER_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
