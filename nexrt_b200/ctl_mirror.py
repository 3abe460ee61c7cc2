"""Host-visible mirror of the control block: the device publishes, the host spins on a flag.

Same scheme as the reference's ``CtlMirror`` (``nex_n2_5_pro/ctl_mirror.py:38-98``): a pinned,
device-mapped ``int32[2][words + 1]`` bank pair; the last node of every captured step copies the
control words into bank ``gen & 1`` and then writes the generation number into the bank's last
word, so the host reads a token without any memcpy, event or stream synchronise.  Here the
publication is folded into the step-end kernel (which also advances the LL sequence) and the
spin runs in native code with the interpreter lock released.
"""

from __future__ import annotations

import ctypes
import time
from typing import List

import numpy as np
import torch

from .ops import lib as L

WAIT_TIMEOUT_S = 120.0


class CtlMirror:
    def __init__(self, device: torch.device, words: int = 32):
        self.words = words
        self.lib = L.load()
        host, dev = ctypes.c_void_p(), ctypes.c_void_p()
        self.nbytes = 2 * (words + 1) * 4
        L.check(self.lib.nexrt_host_mapped_alloc(self.nbytes, ctypes.byref(host), ctypes.byref(dev)), "host_mapped_alloc")
        self._host_ptr, self.dev_ptr = host.value, dev.value
        buf = (ctypes.c_int32 * (2 * (words + 1))).from_address(host.value)
        self.host = np.frombuffer(buf, dtype=np.int32).reshape(2, words + 1)
        self.gen_dev = torch.zeros(1, dtype=torch.int32, device=device)
        self.gen = 0  # generations launched by the host
        # bytes the device writes into host memory per step (control words + generation flag) == bytes a wait() reads back
        self.bytes_per_read = int(self.host[0].nbytes)

    def next_gen(self) -> int:
        self.gen += 1
        return self.gen

    def wait(self, gen: int, timeout_s: float = WAIT_TIMEOUT_S) -> List[int]:
        """Block until generation ``gen`` is published; returns the control words."""
        bank = gen & 1
        flag_addr = self._host_ptr + (bank * (self.words + 1) + self.words) * 4
        rc = self.lib.nexrt_host_wait_flag(ctypes.c_void_p(flag_addr), gen, float(timeout_s))
        if rc != 0:
            raise TimeoutError(f"control mirror: generation {gen} not published within {timeout_s}s")
        return self.host[bank, : self.words].tolist()

    def poll(self, gen: int) -> bool:
        return int(self.host[gen & 1, self.words]) == gen

    def resync(self) -> None:
        """Re-read the device generation (after eager steps or a reset)."""
        self.gen = int(self.gen_dev.item())

    def close(self) -> None:
        if self._host_ptr:
            self.lib.nexrt_host_mapped_free(ctypes.c_void_p(self._host_ptr))
            self._host_ptr = 0
