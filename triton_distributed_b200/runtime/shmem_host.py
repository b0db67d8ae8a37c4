"""Host-side symmetric-memory API with the reference's pynvshmem names.

(reference shmem/nvshmem_bind/pynvshmem/src/pynvshmem.cc:107-215 and python/pynvshmem/__init__.py:93-171.)
There is no NVSHMEM underneath: tensors come from :class:`SymmetricHeap`, "put" is a copy kernel of this
library writing through the peer mapping, signals are 8-byte words in symmetric memory written with
``st.release.sys`` / ``red.release.sys.add`` by a one-thread kernel in stream order, waits are bounded.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
import torch.distributed as dist

from .. import _lib
from .dist import symm_heap
from .heap import SymmTensor
from .status import default_timeout_ns, global_status

NVSHMEM_CMP_EQ, NVSHMEM_CMP_NE, NVSHMEM_CMP_GT, NVSHMEM_CMP_LE, NVSHMEM_CMP_LT, NVSHMEM_CMP_GE = range(6)
NVSHMEM_SIGNAL_SET, NVSHMEM_SIGNAL_ADD = 9, 10


def _stream(device, stream=None) -> int:
    return (stream or torch.cuda.current_stream(device)).cuda_stream


def nvshmem_my_pe() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def nvshmem_n_pes() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def nvshmem_create_tensor(shape: Sequence[int], dtype: torch.dtype) -> SymmTensor:
    """A symmetric tensor: ``.local`` is this rank's copy, ``.peers[r]`` rank r's copy as mapped here."""
    return symm_heap().empty(shape, dtype)


def nvshmem_create_tensor_list_intra_node(shape: Sequence[int], dtype: torch.dtype) -> List[torch.Tensor]:
    """The reference's list form: one tensor per local rank, entry ``rank`` being the local copy."""
    return list(symm_heap().empty(shape, dtype).peers)


symm_tensor = nvshmem_create_tensor


def nvshmem_barrier_all() -> None:
    symm_heap().barrier()


def nvshmem_ptr(t: SymmTensor, pe: int) -> int:
    """Address of rank ``pe``'s copy in this process."""
    return t.ptrs[pe]


def _order_after_current(device, stream) -> None:
    """Make ``stream`` wait for what the current stream has queued (a staging copy made there)."""
    cur = torch.cuda.current_stream(device)
    if stream is not None and stream != cur:
        ev = torch.cuda.Event()
        ev.record(cur)
        stream.wait_event(ev)


def putmem_on_stream(dst: SymmTensor, src: torch.Tensor, pe: int, stream=None) -> None:
    """Copy ``src`` (local) into rank ``pe``'s copy of ``dst``, stream-ordered.

    A non-contiguous ``src`` is first packed on the current stream; ``stream`` is then ordered after that copy."""
    target = dst.peers[pe].reshape(-1).view(torch.uint8)
    if src.numel() * src.element_size() > target.numel():
        raise ValueError("source larger than the symmetric destination")
    if src.device.type != "cuda":
        raise ValueError("putmem_on_stream moves device memory; on CPU use torch.distributed")
    staged = not src.is_contiguous()
    flat = src.contiguous().reshape(-1).view(torch.uint8)
    n = flat.numel()
    if staged:
        _order_after_current(src.device, stream)
        if stream is not None:
            flat.record_stream(stream)
    if n % 16 == 0 and flat.data_ptr() % 16 == 0 and target.data_ptr() % 16 == 0:
        st = global_status()
        _lib.check(_lib.lib().tdist_p2p_copy(flat.data_ptr(), target.data_ptr(), n, 0, min(64, max(1, n // 65536)), 512, 0,
                                             st.device_ptr if st is not None else None, default_timeout_ns(),
                                             _stream(src.device, stream)), "tdist_p2p_copy")
    else:
        with torch.cuda.stream(stream) if stream is not None else _null():
            target[:n].copy_(flat)  # odd sizes: the driver's memcpy


def getmem_on_stream(dst: torch.Tensor, src: SymmTensor, pe: int, stream=None) -> None:
    """Copy rank ``pe``'s copy of ``src`` into the local tensor ``dst``, stream-ordered. ``dst`` must be contiguous
    (a reshaped copy would silently drop the data) and no larger than ``src`` (the read would run past the peer
    mapping)."""
    if not dst.is_contiguous():
        raise ValueError("getmem_on_stream needs a contiguous destination")
    source = src.peers[pe].reshape(-1).view(torch.uint8)
    flat = dst.reshape(-1).view(torch.uint8)
    n = flat.numel()
    if n > source.numel():
        raise ValueError("destination larger than the symmetric source")
    if dst.device.type != "cuda":
        raise ValueError("getmem_on_stream moves device memory; on CPU use torch.distributed")
    if n % 16 == 0 and flat.data_ptr() % 16 == 0 and source.data_ptr() % 16 == 0:
        st = global_status()
        _lib.check(_lib.lib().tdist_p2p_copy(source.data_ptr(), flat.data_ptr(), n, 0, min(64, max(1, n // 65536)), 512, 0,
                                             st.device_ptr if st is not None else None, default_timeout_ns(),
                                             _stream(dst.device, stream)), "tdist_p2p_copy")
    else:
        with torch.cuda.stream(stream) if stream is not None else _null():
            flat.copy_(source[:n])


def signal_op_on_stream(sig: SymmTensor, index: int, value: int, sig_op: int, pe: int, stream=None) -> None:
    """Set (9) or add (10) ``value`` on word ``index`` of rank ``pe``'s copy of the int64 signal array, after
    everything the stream did before."""
    addr = sig.ptrs[pe] + 8 * index
    _lib.check(_lib.lib().tdist_signal_op_on_stream(addr, value, sig_op, _stream(sig.local.device, stream)), "tdist_signal_op_on_stream")


def putmem_signal_on_stream(dst: SymmTensor, src: torch.Tensor, sig: SymmTensor, index: int, value: int, sig_op: int, pe: int,
                            stream=None) -> None:
    """``putmem_on_stream`` followed by the signal: the data is complete at ``pe`` before the signal is."""
    putmem_on_stream(dst, src, pe, stream)
    signal_op_on_stream(sig, index, value, sig_op, pe, stream)


def signal_wait_until_on_stream(sig: SymmTensor, index: int, cmp: int, value: int, stream=None) -> None:
    """Block the stream until the local signal word compares true, with the library's wait limit: on expiry
    the status block records it (``check_status()`` raises) and the stream moves on."""
    st = global_status()
    _lib.check(_lib.lib().tdist_signal_wait_on_stream(sig.local.data_ptr() + 8 * index, cmp, value,
                                                      st.device_ptr if st is not None else None, default_timeout_ns(),
                                                      _stream(sig.local.device, stream)), "tdist_signal_wait_on_stream")


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


# ---------------------------------------------------------------------------- the remaining pynvshmem names
NVSHMEM_TEAM_WORLD, NVSHMEMX_TEAM_NODE = 0, 2


def nvshmem_team_my_pe(team: int = NVSHMEM_TEAM_WORLD) -> int:
    """One NVSwitch node: the node team is the world team."""
    return nvshmem_my_pe()


def nvshmem_team_n_pes(team: int = NVSHMEM_TEAM_WORLD) -> int:
    return nvshmem_n_pes()


def nvshmemx_mc_ptr(team: int, t: SymmTensor) -> int:
    """Address of the multicast alias of ``t`` (0 when the heap was not bound to a multicast object, TDIST_NVLS=1)."""
    return 0 if t.mc is None else t.mc.data_ptr()


def nvshmemx_barrier_all_on_stream(stream=None) -> None:
    from ..ops.collectives import barrier_all_on_stream
    barrier_all_on_stream(stream)


nvshmemx_putmem_on_stream = putmem_on_stream
nvshmemx_putmem_signal_on_stream = putmem_signal_on_stream


def nvshmem_putmem(dst: SymmTensor, src: torch.Tensor, pe: int) -> None:
    """Blocking put: returns when the data is at ``pe``."""
    putmem_on_stream(dst, src, pe)
    torch.cuda.current_stream(src.device).synchronize()


def nvshmem_getmem(dst: torch.Tensor, src: SymmTensor, pe: int) -> None:
    getmem_on_stream(dst, src, pe)
    torch.cuda.current_stream(dst.device).synchronize()


def nvshmem_p(t: SymmTensor, index: int, value, pe: int) -> None:
    """Typed single-element put (``nvshmem_<type>_p``): element ``index`` of rank ``pe``'s copy := value."""
    if t.local.device.type != "cuda":
        t.peers[pe].reshape(-1)[index] = value
        return
    # a device-to-device memcpy of one element (copy engine): no library kernel is handed the peer's memory
    src = torch.tensor([value], dtype=t.local.dtype, device=t.local.device)
    t.peers[pe].reshape(-1)[index:index + 1].copy_(src)


# nvshmem_<type>_p of the reference's host binding (pynvshmem.cc:107-215): the element type comes from the tensor
nvshmem_int_p = nvshmem_int32_p = nvshmem_int64_p = nvshmem_long_p = nvshmem_uint64_p = nvshmem_float_p = nvshmem_p
nvshmem_half_p = nvshmem_bfloat16_p = nvshmem_double_p = nvshmem_p
