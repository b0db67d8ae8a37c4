"""Collectives through the NVSwitch multicast engine (NVLS): ``csrc/kernels/nvls.cu``.

The symmetric heap binds its segments to a multicast object when it is created with
``TDIST_NVLS=1`` (or ``SymmetricHeap(use_nvls=True)``); a :class:`SymmTensor` from such a heap has a
``mc`` alias. ``multimem.st`` to the alias stores into every rank's copy, ``multimem.ld_reduce``
returns the switch-side sum of all copies.

* ``nvls_allgather(buf, ctx)`` — in place, like ``fast_allgather`` (mode ``"nvls"`` /
  ``"push2d_ll_multimem"`` there routes here when the buffer has a multicast alias).
* ``nvls_reduce_scatter(buf, ctx, out)`` — ``out = sum over ranks of buf_r[segment rank]``.
* ``nvls_allreduce(buf, ctx)`` — in place, one shot: every rank reduces its segment through the switch
  and multicasts the result back.

Reference: kernels/nvidia/low_latency_allgather.py:570-697 (the multimem all-gather variant) and
test/nvidia/test_nvshmem_api.py:532-569 (multicast pointers). The reference has no multimem reduction;
NCCL's NVLS algorithms are the baseline for these.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib
from ..runtime import SymmTensor, default_timeout_ns, global_status, symm_heap

NVLS_ALLGATHER, NVLS_REDUCE_SCATTER, NVLS_ALLREDUCE = 0, 1, 2
_DTYPES = {torch.bfloat16: _lib.DT_BF16, torch.float16: _lib.DT_F16, torch.float32: _lib.DT_F32}
launch_count = 0


@dataclass
class NvlsContext:
    rank: int
    world: int
    signal: Optional[SymmTensor] = None      # int64 [2 * MAX_RANKS]: ready flags, done flags
    counters: Optional[torch.Tensor] = None  # int32 [2], local
    epoch: int = 0
    group: object = None


def create_nvls_context(rank: int, world: int, heap=None, group=None, device=None) -> NvlsContext:
    ctx = NvlsContext(rank=rank, world=world, group=group)
    on_cuda = (device is not None and torch.device(device).type == "cuda") or (device is None and torch.cuda.is_available())
    if on_cuda and world > 1:
        heap = heap or symm_heap(group)
        ctx.signal = heap.zeros((2 * _lib.MAX_RANKS,), torch.int64)
        ctx.counters = torch.zeros(2, dtype=torch.int32, device=ctx.signal.local.device)
    return ctx


def nvls_available(buf: SymmTensor) -> bool:
    return buf.mc is not None


def _launch(op: int, buf: SymmTensor, ctx: NvlsContext, out: Optional[torch.Tensor], stream=None) -> None:
    global launch_count
    if buf.mc is None:
        raise _lib.TdistError("this symmetric buffer has no multicast alias: create the heap with TDIST_NVLS=1 on an NVSwitch system")
    local = buf.local
    nbytes = local.numel() * local.element_size()
    if nbytes % (16 * ctx.world):
        raise ValueError("the buffer must split into per-rank segments that are multiples of 16 bytes")
    a = _lib.NvlsArgs()
    a.mc = buf.mc.data_ptr()
    a.local = local.data_ptr()
    a.sig_peer = ctx.signal.cached_ptr_array()
    a.counters = ctx.counters.data_ptr()
    a.output = out.data_ptr() if out is not None else None
    a.seg_bytes = nbytes // ctx.world
    a.world, a.rank, a.op = ctx.world, ctx.rank, op
    a.dtype = _DTYPES.get(local.dtype, _lib.DT_F32)
    ctx.epoch += 1
    a.epoch = ctx.epoch
    st = global_status()
    a.status = st.device_ptr if st is not None else None
    a.timeout_ns = default_timeout_ns()
    a.stream = (stream or torch.cuda.current_stream(local.device)).cuda_stream
    _lib.check(_lib.lib().tdist_nvls(C.byref(a)), "tdist_nvls")
    launch_count += 1


def nvls_allgather(buf: SymmTensor, ctx: NvlsContext, stream=None) -> torch.Tensor:
    """In place: rank r has written segment r of its copy; afterwards every copy holds all segments."""
    local = buf.local
    if local.device.type != "cuda":
        if ctx.world > 1:
            flat = local.reshape(-1).view(torch.uint8)
            seg = flat.numel() // ctx.world
            dist.all_gather_into_tensor(flat, flat[ctx.rank * seg:(ctx.rank + 1) * seg].clone(), group=ctx.group)
        return local
    if ctx.world > 1:
        _launch(NVLS_ALLGATHER, buf, ctx, None, stream)
    return local


def nvls_reduce_scatter(buf: SymmTensor, ctx: NvlsContext, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """``out`` (1/world of the buffer) = sum over ranks of their copies' segment ``rank``; fp32 accumulation
    inside the switch for bf16 / fp16."""
    local = buf.local
    flat = local.reshape(-1)
    seg = flat.numel() // ctx.world
    if local.device.type != "cuda" or ctx.world == 1:
        acc = flat.float() if local.dtype in (torch.bfloat16, torch.float16) else flat.clone()
        if ctx.world > 1:
            dist.all_reduce(acc, group=ctx.group)
        res = acc[ctx.rank * seg:(ctx.rank + 1) * seg].to(local.dtype)
        if out is not None:
            out.reshape(-1).copy_(res)
            return out
        return res
    if local.dtype not in _DTYPES:
        raise TypeError(f"NVLS reductions take {list(_DTYPES)}, got {local.dtype}")
    o = out if out is not None else torch.empty(seg, dtype=local.dtype, device=local.device)
    _launch(NVLS_REDUCE_SCATTER, buf, ctx, o, stream)
    return o


def nvls_allreduce(buf: SymmTensor, ctx: NvlsContext, stream=None) -> torch.Tensor:
    """In place: every copy ends up holding the sum of all copies."""
    local = buf.local
    if local.device.type != "cuda" or ctx.world == 1:
        if ctx.world > 1:
            acc = local.float() if local.dtype in (torch.bfloat16, torch.float16) else local
            dist.all_reduce(acc, group=ctx.group)
            local.copy_(acc.to(local.dtype))
        return local
    if local.dtype not in _DTYPES:
        raise TypeError(f"NVLS reductions take {list(_DTYPES)}, got {local.dtype}")
    _launch(NVLS_ALLREDUCE, buf, ctx, None, stream)
    return local
