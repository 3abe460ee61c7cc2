"""Symmetric device memory: one buffer per rank, every rank knows every peer's address and
(when NVSwitch multicast is available) one multicast address that replicates a store to all.

Primary substrate is ``torch.distributed._symmetric_memory`` exactly as in the reference
(``symm_mem.empty`` + ``rendezvous`` -> ``buffer_ptrs`` / ``multicast_ptr``,
``nex_n2_5_pro/gdn.py:178-198``).  Two differences: a missing multicast address is not fatal
(the LL channel then publishes with one unicast store per peer), and if symmetric memory
cannot be created at all the buffer falls back to ``cudaMalloc`` + CUDA IPC handles exchanged
over the process group (``csrc/host_runtime.cu``).

``NEXRT_SYMM`` selects the substrate: ``auto`` (default), ``torch``, ``ipc``.
``NEXRT_NO_MULTICAST=1`` ignores the multicast address (used by failure tests, where a rank
may leave while its memory is bound to a multicast object).
"""

from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist


class SymmetricBuffer:
    """``nbytes`` of zero-initialised device memory on every rank of ``group``."""

    def __init__(self, nbytes: int, device: torch.device, group=None, world: int = 1, rank: int = 0):
        self.nbytes = int(nbytes)
        self.device = device
        self.world = world
        self.rank = rank
        self.mc_ptr = 0
        self.peer_ptrs: List[int] = []
        self.backend = "local"
        self._keep = []
        if world == 1:
            self.tensor = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)
            self.peer_ptrs = [self.tensor.data_ptr()]
            return
        mode = os.environ.get("NEXRT_SYMM", "auto")
        err: Optional[Exception] = None
        if mode in ("auto", "torch"):
            try:
                self._init_torch(group)
                return
            except Exception as e:  # noqa: BLE001 - any failure selects the fallback
                err = e
                if mode == "torch":
                    raise
        self._init_ipc(group, err)

    # ---- torch symmetric memory (NVLS multicast when the fabric offers it) ------------------
    def _init_torch(self, group) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        t = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        hdl = symm_mem.rendezvous(t, group if group is not None else dist.group.WORLD)
        t.zero_()
        self.tensor = t
        self.peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        if os.environ.get("NEXRT_NO_MULTICAST") == "1":
            mc = 0
        self.mc_ptr = mc
        self.backend = "torch-symm"
        self._keep.append(hdl)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    # ---- CUDA IPC fallback -------------------------------------------------------------------
    def _init_ipc(self, group, why: Optional[Exception]) -> None:
        from ..ops import lib as L

        lib = L.load()
        p = ctypes.c_void_p()
        L.check(lib.nexrt_ipc_alloc(self.nbytes, ctypes.byref(p)), "ipc_alloc")
        handle = (ctypes.c_ubyte * 64)()
        L.check(lib.nexrt_ipc_get_handle(p, handle), "ipc_get_handle")
        mine = torch.tensor(list(bytes(handle)), dtype=torch.uint8, device=self.device)
        gathered = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(gathered, mine, group=group)
        self.peer_ptrs = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                self.peer_ptrs.append(p.value)
                continue
            raw = (ctypes.c_ubyte * 64)(*h.cpu().tolist())
            q = ctypes.c_void_p()
            L.check(lib.nexrt_ipc_open(raw, ctypes.byref(q)), "ipc_open")
            self.peer_ptrs.append(q.value)
        self._raw = p.value
        self.tensor = _tensor_from_ptr(p.value, self.nbytes, self.device)
        self.backend = "cuda-ipc"
        self.fallback_reason = repr(why) if why else ""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    @property
    def local_ptr(self) -> int:
        return self.peer_ptrs[self.rank] if self.world > 1 else self.tensor.data_ptr()


def _tensor_from_ptr(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    """View raw device memory as a uint8 tensor (zero copy) through the CUDA array interface."""

    class _Holder:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}

    return torch.as_tensor(_Holder(), device=device)
