"""Host handles for the device primitives: each primitive of ``csrc/device/signal.cuh`` /
``shmem.cuh`` can be run on its own through a tiny kernel (``csrc/kernels/primitives.cu``).

This is the Python face of what the reference exposes as a device language
(``triton_dist.language``: wait / consume_token / notify / symm_at / rank / num_ranks, reference
python/triton_dist/language.py:57-112; ``libshmem_device``: put / get / signal / barrier / broadcast /
fcollect, reference patches/triton/python/triton/language/extra/libshmem_device.py:28-260). Kernels written
against this library include the headers and call the device functions directly; the handles below
exist for tests, bring-up on a new machine, and as executable documentation of the protocols.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from .. import _lib
from ..runtime import SymmTensor, default_timeout_ns, global_status, symm_heap

OPS = {
    "ring_put": _lib.PRIM_RING_PUT, "notify_wait": _lib.PRIM_NOTIFY_WAIT, "notify_add": _lib.PRIM_NOTIFY_ADD,
    "put_signal": _lib.PRIM_PUT_SIGNAL, "put_quiet_signal": _lib.PRIM_PUT_QUIET_SIGNAL, "get": _lib.PRIM_GET,
    "broadcast": _lib.PRIM_BROADCAST, "fcollect": _lib.PRIM_FCOLLECT, "grid_barrier": _lib.PRIM_GRID_BARRIER, "scoped_ops": _lib.PRIM_SCOPED_OPS,
    "barrier": _lib.PRIM_BARRIER,            # `value` rounds of barrier_all at the requested scope
    "bounds_probe": _lib.PRIM_BOUNDS_PROBE,  # bounds-checked build only: out-of-range accesses that must be recorded and skipped
}
SCOPES = {"thread": 0, "warp": 1, "block": 2}

# the reference's NVSHMEM constants, for code that spells them out
NVSHMEM_CMP_EQ, NVSHMEM_CMP_NE, NVSHMEM_CMP_GT, NVSHMEM_CMP_LE, NVSHMEM_CMP_LT, NVSHMEM_CMP_GE = range(6)
NVSHMEM_SIGNAL_SET, NVSHMEM_SIGNAL_ADD = 9, 10


@dataclass
class PrimitiveContext:
    rank: int
    world: int
    nbytes: int
    data: SymmTensor            # uint8 [(world + 2) * nbytes]: slots 0..world-1 receive, slot `world` is the source
    sig: SymmTensor             # int64 [16]
    result: torch.Tensor        # int32 [8]
    grid_counter: torch.Tensor  # int32 [1]
    barrier_epoch: torch.Tensor # int64 [1]

    def slot(self, s: int) -> torch.Tensor:
        return self.data.local[s * self.nbytes:(s + 1) * self.nbytes]

    @property
    def source(self) -> torch.Tensor:
        return self.slot(self.world)


def create_primitive_context(rank: int, world: int, nbytes: int = 4096, heap=None, group=None) -> PrimitiveContext:
    heap = heap or symm_heap(group)
    data = heap.zeros(((world + 2) * nbytes,), torch.uint8)
    sig = heap.zeros((16,), torch.int64)
    dev = data.local.device
    return PrimitiveContext(rank, world, nbytes, data, sig, torch.zeros(8, dtype=torch.int32, device=dev),
                            torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int64, device=dev))


def run_primitive(ctx: PrimitiveContext, op: str, value: int = 1, phase: int = 3, scope: str = "block", grid: int = 64,
                  stream=None) -> torch.Tensor:
    """Launch the test kernel of ``op`` (see ``OPS``) and return the context's result tensor
    (filled asynchronously on the stream)."""
    a = _lib.PrimArgs()
    a.data_peer = ctx.data.cached_ptr_array()
    a.sig_peer = ctx.sig.cached_ptr_array()
    a.result = ctx.result.data_ptr()
    a.grid_counter = ctx.grid_counter.data_ptr()
    a.barrier_epoch = ctx.barrier_epoch.data_ptr()
    a.world, a.rank, a.op, a.phase, a.nbytes = ctx.world, ctx.rank, OPS[op], phase, ctx.nbytes
    a.scope, a.grid, a.value = SCOPES[scope], grid, value
    st = global_status()
    a.status = st.device_ptr if st is not None else None
    a.timeout_ns = default_timeout_ns()
    a.stream = (stream or torch.cuda.current_stream(ctx.result.device)).cuda_stream
    _lib.check(_lib.lib().tdist_primitive(C.byref(a)), "tdist_primitive")
    return ctx.result
