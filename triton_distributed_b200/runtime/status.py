"""Host view of the device status block that bounded waits report into.

The reference has nothing of the kind: its waits spin without limit
(reference patches/triton/third_party/nvidia/lib/TritonNVIDIAGPUToLLVM/DistributedOpToLLVM.cpp:198-201).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from .. import _lib

_CODES = {0: "ok", 1: "flag wait timed out", 2: "mbarrier wait timed out", 3: "bad argument"}
_KERNELS = {1: "gemm_sm100", 2: "collectives", 3: "a2a", 4: "flash_decode", 5: "primitives", 6: "moe"}


def default_timeout_ns() -> int:
    return int(float(os.environ.get("TDIST_WAIT_TIMEOUT_MS", "4000")) * 1e6)


class StatusBlock:
    """One per process. ``device_ptr`` goes into kernel arguments; :meth:`check` is called after
    the stream has been synchronised and raises :class:`TdistTimeoutError` if any wait gave up."""

    def __init__(self):
        self._host = C.POINTER(_lib.Status)()
        dptr = C.c_void_p()
        _lib.check(_lib.lib().tdist_status_create(C.byref(self._host), C.byref(dptr)), "tdist_status_create")
        self.device_ptr = dptr.value

    @property
    def record(self) -> "_lib.Status":
        return self._host.contents

    def aborted(self) -> bool:
        return self.record.abort_flag != 0

    def describe(self) -> str:
        s = self.record
        return (f"{_CODES.get(s.code, s.code)} in kernel {_KERNELS.get(s.kernel_id, s.kernel_id)} on rank {s.rank} "
                f"(block {s.block}, site {s.where}): peer {s.peer}, index {s.index}, expected {s.expected}, seen {s.seen}")

    def reset(self) -> None:
        C.memset(self._host, 0, C.sizeof(_lib.Status))

    def check(self, reset: bool = True) -> None:
        if self.aborted():
            msg = self.describe()
            if reset:
                self.reset()
            raise _lib.TdistTimeoutError(msg)


_GLOBAL: Optional[StatusBlock] = None


def global_status() -> Optional[StatusBlock]:
    """Process-wide status block (``None`` when there is no GPU)."""
    global _GLOBAL
    if _GLOBAL is None and torch.cuda.is_available():
        _GLOBAL = StatusBlock()
    return _GLOBAL


def check_status(synchronize: bool = True) -> None:
    """Synchronise the device and raise if a bounded wait reported a timeout."""
    st = global_status()
    if st is None:
        return
    if synchronize:
        torch.cuda.synchronize()
    st.check()
