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
_KERNELS = {1: "gemm_sm100", 2: "collectives", 3: "a2a", 4: "flash_decode", 5: "primitives", 6: "moe", 7: "moe_ep", 8: "bounds check"}


_TIMEOUT_CACHE = [None, 0]


def default_timeout_ns() -> int:
    """Limit of every bounded device wait, from TDIST_WAIT_TIMEOUT_MS (default 4 s); the parsed value is
    cached per distinct setting because this sits on every launch path."""
    raw = os.environ.get("TDIST_WAIT_TIMEOUT_MS", "4000")
    if _TIMEOUT_CACHE[0] != raw:
        _TIMEOUT_CACHE[0] = raw
        _TIMEOUT_CACHE[1] = int(float(raw) * 1e6)
    return _TIMEOUT_CACHE[1]


class StatusBlock:
    """One per process, in device memory. ``device_ptr`` goes into kernel arguments; :meth:`check`
    is called after the stream has been synchronised, copies the block back and raises
    :class:`TdistTimeoutError` if any wait gave up."""

    def __init__(self):
        dptr = C.c_void_p()
        _lib.check(_lib.lib().tdist_status_create(C.byref(dptr)), "tdist_status_create")
        self.device_ptr = dptr.value
        self.aborts = 0   # reports raised so far: kernels cut short may have left in-kernel counters mid-count

    @property
    def record(self) -> "_lib.Status":
        """Snapshot of the block (blocking device-to-host copy)."""
        rec = _lib.Status()
        _lib.check(_lib.lib().tdist_status_read(self.device_ptr, C.byref(rec)), "tdist_status_read")
        return rec

    def aborted(self) -> bool:
        return self.record.abort_flag != 0

    @staticmethod
    def _describe(s) -> str:
        return (f"{_CODES.get(s.code, s.code)} in kernel {_KERNELS.get(s.kernel_id, s.kernel_id)} on rank {s.rank} "
                f"(block {s.block}, site {s.where}): peer {s.peer}, index {s.index}, expected {s.expected}, seen {s.seen}")

    def describe(self) -> str:
        return self._describe(self.record)

    def reset(self) -> None:
        _lib.check(_lib.lib().tdist_status_reset(self.device_ptr), "tdist_status_reset")

    def check(self, reset: bool = True) -> None:
        rec = self.record
        if rec.abort_flag != 0:
            self.aborts += 1
            if reset:
                self.reset()
            raise _lib.TdistTimeoutError(self._describe(rec))


_GLOBAL: Optional[StatusBlock] = None


def counters_clean(t: torch.Tensor, start: int = 0) -> None:
    """Some kernels keep arrival counters in device memory and leave them at zero when they finish. A launch that was
    cut short by a reported wait may have left them mid-count: the first use of ``t`` after such a report zeroes
    ``t[start:]`` again (an integer comparison on every other call)."""
    st = global_status()
    gen = st.aborts if st is not None else 0
    if getattr(t, "_tdist_abort_gen", gen) != gen:
        t[start:].zero_()
    t._tdist_abort_gen = gen


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
