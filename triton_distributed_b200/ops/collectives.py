"""Standalone collectives on symmetric buffers and the host-side stream primitives.

Public surface (names and argument conventions of the reference):

* ``barrier_all_on_stream``, ``wait_eq``, ``set_signal``
  (reference python/triton_dist/kernels/nvidia/common_ops.py:162-211)
* ``create_fast_allgather_context`` / ``fast_allgather(symm_buffer, ctx, mode=...)`` — in place on a
  symmetric byte buffer, rank r's segment at ``r * nbytes / world``
  (reference kernels/nvidia/low_latency_allgather.py:781-990)
* ``AllGatherMethod``, ``get_auto_all_gather_method``, ``cp_engine_producer_all_gather_intra_node``
  — the copy-engine variant kept as a baseline (reference kernels/nvidia/allgather.py:44-135,261-288)
* ``create_reduce_scater_2d_ctx`` / ``reduce_scatter_2d_op(input[M,N], ctx) -> [M/ws, N]``, ``ring_reduce``
  (reference kernels/nvidia/reduce_scatter.py:143-183,752-799)

On CUDA every collective is one kernel launch from ``csrc/kernels/collectives.cu``; on CPU tensors
the same functions go through ``torch.distributed`` (gloo), which is also the test oracle.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _lib
from ..utils.profile import nvtx_range
from ..runtime import SymmTensor, default_timeout_ns, global_status, symm_heap

launch_count = 0

_AG_MODES = {
    "pull": _lib.AG_PULL,
    "push_ordered": _lib.AG_PUSH_ORDERED,   # all copy CTAs serve rank - 1 first, then rank - 2, ...: segments land one by one
    "push": _lib.AG_PUSH, "push2d": _lib.AG_PUSH, "push3d": _lib.AG_PUSH, "push_numa_2d": _lib.AG_PUSH,
    "ll": _lib.AG_LL, "push2d_ll": _lib.AG_LL, "push3d_ll": _lib.AG_LL, "push_numa_2d_ll": _lib.AG_LL,
    "push_numa_2d_ll_multinode": _lib.AG_LL, "push2d_ll_multimem": _lib.AG_LL, "nvls": _lib.AG_LL,
}
_NVLS_MODES = ("push2d_ll_multimem", "nvls")  # served by multimem.st when the buffer has a multicast alias, else by LL
_RS_DTYPES = {torch.bfloat16: _lib.DT_BF16, torch.float16: _lib.DT_F16, torch.float32: _lib.DT_F32, torch.int32: _lib.DT_I32}


def _status_ptr():
    st = global_status()
    return st.device_ptr if st is not None else None


def _stream_ptr(device, stream=None):
    return (stream or torch.cuda.current_stream(device)).cuda_stream


# ---------------------------------------------------------------------------- barrier / flags
@dataclass
class BarrierContext:
    """Symmetric flag array and local epoch counter of the device-side barrier."""

    flags: SymmTensor          # int64 [8]
    epoch: torch.Tensor        # int64 [1], local
    rank: int
    world: int
    group: object = None


_BARRIER: Optional[BarrierContext] = None


def create_barrier_context(heap=None, group=None) -> BarrierContext:
    heap = heap or symm_heap(group)
    flags = heap.zeros((_lib.MAX_RANKS,), torch.int64)
    epoch = torch.zeros(1, dtype=torch.int64, device=flags.local.device)
    return BarrierContext(flags, epoch, heap.rank, heap.world, group)


def barrier_all_on_stream(stream=None, is_intra_node: bool = True, symm_barrier_buf=None, local_world_size: int = 0,
                          barrier_value: int = 1, ctx: Optional[BarrierContext] = None) -> None:
    """Barrier of all ranks, ordered on ``stream`` (no host synchronisation): work enqueued after
    it on any rank starts after the work enqueued before it on every rank. The reference's extra
    arguments are accepted and ignored (one node, one barrier kernel)."""
    global _BARRIER, launch_count
    if not torch.cuda.is_available():
        if dist.is_initialized():
            dist.barrier()
        return
    if ctx is None:
        if _BARRIER is None:
            _BARRIER = create_barrier_context()
        ctx = _BARRIER
    if ctx.world == 1:
        return
    dev = ctx.flags.local.device
    arr = (C.c_void_p * _lib.MAX_RANKS)(*[C.c_void_p(p) for p in ctx.flags.ptrs])
    _lib.check(_lib.lib().tdist_barrier_all(arr, C.c_void_p(ctx.epoch.data_ptr()), ctx.world, ctx.rank,
                                            C.c_void_p(_status_ptr()), C.c_uint64(default_timeout_ns()),
                                            C.c_void_p(_stream_ptr(dev, stream))), "tdist_barrier_all")
    launch_count += 1


def set_signal(ptr: int, signal: int, stream=None, require_i64: bool = False) -> None:
    """Stream-ordered write of ``signal`` to the 32/64-bit word at device address ``ptr``
    (``cuStreamWriteValue``)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    _lib.check(_lib.lib().tdist_stream_write_value(C.c_void_p(_stream_ptr(dev, stream)), C.c_uint64(ptr),
                                                   C.c_uint64(signal), int(require_i64)), "set_signal")


def wait_eq(ptr: int, signal: int, stream=None, require_i64: bool = False) -> None:
    """Make ``stream`` wait until the word at ``ptr`` equals ``signal`` (``cuStreamWaitValue``).
    The wait itself has no time limit: only use it for a value that is certain to be written."""
    dev = torch.device("cuda", torch.cuda.current_device())
    _lib.check(_lib.lib().tdist_stream_wait_value(C.c_void_p(_stream_ptr(dev, stream)), C.c_uint64(ptr),
                                                  C.c_uint64(signal), int(require_i64), 0), "wait_eq")


# ---------------------------------------------------------------------------- all-gather
class AllGatherMethod(enum.Enum):
    Auto = 0
    All2All_IntraNode = 1
    All2All_InterNode = 2
    Ring1D_IntraNode = 3
    Ring2D_IntraNode = 4
    Ring2D_InterNode = 5


def get_auto_all_gather_method(num_ranks: int, num_local_ranks: int) -> AllGatherMethod:
    """NVSwitch node: every peer is one hop away, so full-mesh is always the choice."""
    return AllGatherMethod.All2All_IntraNode if num_ranks <= num_local_ranks else AllGatherMethod.All2All_InterNode


def cp_engine_producer_all_gather_intra_node(rank: int, num_ranks: int, local_tensor: torch.Tensor,
                                             remote_tensor_buffers: List[torch.Tensor], barrier_buffers=None,
                                             stream=None, for_correctness: bool = False,
                                             all_gather_method: AllGatherMethod = AllGatherMethod.Auto) -> None:
    """Copy-engine full-mesh pull: for every peer, ``cudaMemcpyAsync`` its segment out of its
    buffer into ``remote_tensor_buffers[rank]`` on ``stream``. Baseline for the in-kernel paths;
    the caller is responsible for the peers' segments being ready (e.g. ``barrier_all_on_stream``)."""
    rows = local_tensor.shape[0]
    mine = remote_tensor_buffers[rank]
    with torch.cuda.stream(stream or torch.cuda.current_stream()):
        mine[rank * rows:(rank + 1) * rows].copy_(local_tensor)
        for step in range(1, num_ranks):
            src = (rank + step) % num_ranks
            mine[src * rows:(src + 1) * rows].copy_(remote_tensor_buffers[src][src * rows:(src + 1) * rows])


@dataclass
class FastAllGatherContext:
    rank: int
    world: int
    max_buffer_size: int
    signal: Optional[SymmTensor] = None       # int64 [8]
    ll_buffer: Optional[SymmTensor] = None    # uint8 [2 * 2 * ll_max]: two parities of LL packets
    ll_max: int = 0                           # largest buffer the LL path serves (larger ones are pushed)
    counters: Optional[torch.Tensor] = None   # int32 [8], local
    epoch: int = 0
    ctas_per_peer: int = 0
    group: object = None
    nvls: object = None                       # NvlsContext, created on the first multimem call
    _ll_arrays: object = None


def create_fast_allgather_context(rank: int, node: int = 0, num_ranks: int = 1, num_nodes: int = 1,
                                  max_buffer_size: int = 2 * 32 * 1024 * 1024, heap=None, group=None,
                                  device=None) -> FastAllGatherContext:
    ctx = FastAllGatherContext(rank=rank, world=num_ranks, max_buffer_size=max_buffer_size, group=group)
    on_cuda = (device is not None and torch.device(device).type == "cuda") or (device is None and torch.cuda.is_available())
    if on_cuda and num_ranks > 1:
        heap = heap or symm_heap(group)
        ctx.signal = heap.zeros((_lib.MAX_RANKS,), torch.int64)
        ctx.ll_max = min(max_buffer_size, 8 << 20)
        ctx.ll_buffer = heap.zeros((4 * ctx.ll_max,), torch.uint8)
        ctx.counters = torch.zeros(_lib.MAX_RANKS, dtype=torch.int32, device=ctx.signal.local.device)
    return ctx


@nvtx_range("tdist.fast_allgather")
def fast_allgather(symm_buffer: SymmTensor, ctx: Optional[FastAllGatherContext] = None, rank: Optional[int] = None,
                   node: int = 0, num_ranks: Optional[int] = None, num_nodes: int = 1, mode: str = "pull",
                   phase: int = 3, stream=None) -> torch.Tensor:
    """In-place all-gather of a symmetric buffer: on entry rank r has written its own segment
    (bytes ``[r*seg, (r+1)*seg)`` with ``seg = nbytes / world``); on return (stream-ordered) the
    local copy holds every rank's segment. The buffer must not be rewritten by any rank before all
    ranks have finished reading the previous result (use distinct buffers or a barrier)."""
    global launch_count
    local = symm_buffer.local
    if ctx is None:
        ctx = create_fast_allgather_context(rank, node, num_ranks, num_nodes, max_buffer_size=local.numel() * local.element_size())
    if mode not in _AG_MODES:
        raise ValueError(f"unknown all-gather mode {mode!r}; known: {sorted(_AG_MODES)}")
    nbytes = local.numel() * local.element_size()
    if nbytes % ctx.world:
        raise ValueError("buffer size must be divisible by the world size")
    if local.device.type != "cuda":
        if ctx.world > 1:
            flat = local.reshape(-1).view(torch.uint8)
            seg = nbytes // ctx.world
            mine = flat[ctx.rank * seg:(ctx.rank + 1) * seg].clone()
            dist.all_gather_into_tensor(flat, mine, group=ctx.group)
        return local
    if ctx.world == 1:
        return local
    if nbytes > ctx.max_buffer_size:
        raise ValueError(f"buffer of {nbytes} bytes exceeds the context's max_buffer_size {ctx.max_buffer_size}")
    if mode in _NVLS_MODES and symm_buffer.mc is not None and phase == 3 and (nbytes // ctx.world) % 16 == 0:
        from . import nvls as NV
        if ctx.nvls is None:
            ctx.nvls = NV.create_nvls_context(ctx.rank, ctx.world, group=ctx.group, device=local.device)
        return NV.nvls_allgather(symm_buffer, ctx.nvls, stream=stream)
    a = _lib.CollArgs()
    a.buf_peer = symm_buffer.cached_ptr_array()
    a.sig_peer = ctx.signal.cached_ptr_array()
    a.counters = ctx.counters.data_ptr()
    a.seg_bytes = nbytes // ctx.world
    a.world, a.rank = ctx.world, ctx.rank
    a.mode = _AG_MODES[mode]
    if a.mode == _lib.AG_LL and (nbytes > ctx.ll_max or (nbytes // ctx.world) % 8):
        # LL doubles the bytes on the wire (only worth it for small messages) and moves 8-byte words
        a.mode = _lib.AG_PUSH
    a.phase = phase
    a.ctas_per_peer = ctx.ctas_per_peer or (1 if a.seg_bytes <= (64 << 10) else (4 if a.seg_bytes <= (4 << 20) else 16))
    if phase != 2:
        ctx.epoch += 1
    a.epoch = ctx.epoch
    half_bytes = 2 * ctx.ll_max
    if ctx._ll_arrays is None:
        ctx._ll_arrays = tuple(_lib.ptr_array([p + h * half_bytes for p in ctx.ll_buffer.ptrs]) for h in range(2))
    a.ll_peer = ctx._ll_arrays[ctx.epoch & 1]
    a.status = _status_ptr()
    a.timeout_ns = default_timeout_ns()
    a.stream = _stream_ptr(local.device, stream)
    _lib.check(_lib.lib().tdist_allgather(C.byref(a)), "tdist_allgather")
    launch_count += 1
    return local


# ---------------------------------------------------------------------------- reduce-scatter
@dataclass
class ReduceScatter2DContext:
    max_M: int
    N: int
    rank: int
    world: int
    dtype: torch.dtype
    staging: Optional[SymmTensor] = None      # [2, world * max_M/world * N]
    signal: Optional[SymmTensor] = None
    counters: Optional[torch.Tensor] = None
    epoch: int = 0
    ctas_per_peer: int = 0
    group: object = None


def create_reduce_scater_2d_ctx(max_M: int, N: int, rank: int, world_size: int, local_world_size: Optional[int] = None,
                                dtype: torch.dtype = torch.bfloat16, overlap_with_gemm: bool = True,
                                num_reduction_sms: int = 15, heap=None, group=None, device=None) -> ReduceScatter2DContext:
    """(The reference spells it ``scater``.) Allocates double-buffered staging ``[2, max_M, N]`` that
    peers scatter into, and the arrival flags."""
    ctx = ReduceScatter2DContext(max_M=max_M, N=N, rank=rank, world=world_size, dtype=dtype, group=group)
    on_cuda = (device is not None and torch.device(device).type == "cuda") or (device is None and torch.cuda.is_available())
    if on_cuda:
        heap = heap or symm_heap(group)
        ctx.staging = heap.empty((2, max_M * N), dtype)
        ctx.signal = heap.zeros((_lib.MAX_RANKS,), torch.int64)
        ctx.counters = torch.zeros(_lib.MAX_RANKS, dtype=torch.int32, device=ctx.signal.local.device)
    return ctx


create_reduce_scatter_2d_ctx = create_reduce_scater_2d_ctx


@nvtx_range("tdist.reduce_scatter_2d_op")
def reduce_scatter_2d_op(input: torch.Tensor, ctx: ReduceScatter2DContext, out: Optional[torch.Tensor] = None,
                         phase: int = 3, stream=None) -> torch.Tensor:
    """``out[M/ws, N] = sum over ranks of input_r[rank*M/ws:(rank+1)*M/ws]`` (fp32 accumulation for
    floating types, exact for int32)."""
    global launch_count
    M, N = input.shape
    if M % ctx.world:
        raise ValueError("M must be divisible by the world size")
    mpr = M // ctx.world
    if input.device.type != "cuda":
        acc = input.to(torch.float32) if input.dtype in (torch.bfloat16, torch.float16) else input.clone()
        if ctx.world > 1:
            dist.all_reduce(acc, group=ctx.group)
        return acc[ctx.rank * mpr:(ctx.rank + 1) * mpr].to(input.dtype)
    if ctx.world == 1:   # one rank: the reduce-scatter of a single contribution is a copy
        if out is not None:
            out.copy_(input)
            return out
        return input.clone()
    if input.dtype not in _RS_DTYPES:
        raise TypeError(f"reduce-scatter supports {list(_RS_DTYPES)}, got {input.dtype}")
    if not input.is_contiguous():
        raise ValueError("input must be contiguous")
    esize = input.element_size()
    seg_bytes = mpr * N * esize
    if seg_bytes % 16:
        raise ValueError("rows per rank * N * element size must be a multiple of 16 bytes")
    if M * N > ctx.max_M * ctx.N:
        raise ValueError("input exceeds the context's staging")
    o = out if out is not None else torch.empty((mpr, N), dtype=input.dtype, device=input.device)
    a = _lib.CollArgs()
    half = (ctx.epoch + (1 if phase != 2 else 0)) & 1
    a.buf_peer = ctx.staging.half_ptr_arrays()[half]
    a.sig_peer = ctx.signal.cached_ptr_array()
    a.counters = ctx.counters.data_ptr()
    a.input = input.data_ptr()
    a.output = o.data_ptr()
    a.seg_bytes = seg_bytes
    a.world, a.rank = ctx.world, ctx.rank
    a.phase = phase
    a.dtype = _RS_DTYPES[input.dtype]
    a.ctas_per_peer = ctx.ctas_per_peer or (1 if seg_bytes <= (64 << 10) else (4 if seg_bytes <= (4 << 20) else 16))
    if phase != 2:
        ctx.epoch += 1
    a.epoch = ctx.epoch
    a.status = _status_ptr()
    a.timeout_ns = default_timeout_ns()
    a.stream = _stream_ptr(input.device, stream)
    _lib.check(_lib.lib().tdist_reduce_scatter(C.byref(a)), "tdist_reduce_scatter")
    launch_count += 1
    return o


def topk_reduce_scatter(y_sorted: torch.Tensor, pos_of: torch.Tensor, weights: Optional[torch.Tensor], ntok: int, topk: int,
                        ctx: ReduceScatter2DContext, out: Optional[torch.Tensor] = None, phase: int = 3, stream=None) -> torch.Tensor:
    """Fused MoE tail: ``out[M/ws, N] = rows of this rank of sum_ranks P_r`` with
    ``P_r[t] = sum_k weights[t,k] * y_sorted_r[pos_of[t*topk+k]]``. ``P_r`` is never materialised: the kernel reduces
    the top-k expert outputs of each token straight into the owning rank's staging, signals, then sums the
    sources in fp32 (reference kernels/nvidia/moe_reduce_rs.py:471-546, the kernel that stores into peers from
    inside the reduction)."""
    global launch_count
    N = y_sorted.shape[1]
    if ntok % ctx.world:
        raise ValueError("the token count must be divisible by the world size")
    mpr = ntok // ctx.world
    if y_sorted.device.type != "cuda" or y_sorted.dtype != torch.bfloat16:
        rows = y_sorted[pos_of.long()].float().view(ntok, topk, N)
        w = weights.float().view(ntok, topk, 1) if weights is not None else 1.0
        return reduce_scatter_2d_op((rows * w).sum(1).to(y_sorted.dtype), ctx, out=out, phase=phase, stream=stream)
    if ctx.world == 1:   # nothing to scatter: the top-k reduce kernel on the whole GPU
        from .moe_tp import topk_reduce
        res = topk_reduce(y_sorted, pos_of, weights, ntok, topk)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if not y_sorted.is_contiguous() or (N * 2) % 16:
        raise ValueError("y_sorted must be contiguous with N a multiple of 8")
    if ntok * N > ctx.max_M * ctx.N:
        raise ValueError("problem exceeds the context's staging")
    o = out if out is not None else torch.empty((mpr, N), dtype=y_sorted.dtype, device=y_sorted.device)
    a = _lib.CollArgs()
    half = (ctx.epoch + (1 if phase != 2 else 0)) & 1
    a.buf_peer = ctx.staging.half_ptr_arrays()[half]
    a.sig_peer = ctx.signal.cached_ptr_array()
    a.counters = ctx.counters.data_ptr()
    a.input = y_sorted.data_ptr()
    a.output = o.data_ptr()
    a.seg_bytes = mpr * N * 2
    a.world, a.rank = ctx.world, ctx.rank
    a.phase = phase
    a.dtype = _lib.DT_BF16
    # the send half computes the top-k sums of the peers' rows: spread it over the whole GPU
    a.ctas_per_peer = ctx.ctas_per_peer or max(1, min(128, 144 // max(1, ctx.world - 1)))
    pos = pos_of if pos_of.dtype == torch.int32 else pos_of.to(torch.int32)
    w = weights.float().contiguous() if weights is not None else None
    a.pos_of = pos.contiguous().data_ptr()
    a.topk_w = w.data_ptr() if w is not None else None
    a.topk, a.row_bytes = topk, N * 2
    if phase != 2:
        ctx.epoch += 1
    a.epoch = ctx.epoch
    a.status = _status_ptr()
    a.timeout_ns = default_timeout_ns()
    a.stream = _stream_ptr(y_sorted.device, stream)
    _lib.check(_lib.lib().tdist_reduce_scatter(C.byref(a)), "tdist_reduce_scatter")
    launch_count += 1
    return o


def ring_reduce(input: torch.Tensor, output: torch.Tensor, begin_idx: int, num_splits: int, num_sms: int = -1) -> torch.Tensor:
    """Sum the ``num_splits`` row blocks of ``input`` (starting the rotation at ``begin_idx``) into
    ``output``; accumulation in fp32 (reference kernels/nvidia/reduce_scatter.py:752-763)."""
    global launch_count
    M = input.shape[0] // num_splits
    block_bytes = M * (input.numel() // max(1, input.shape[0])) * input.element_size()
    if (input.device.type == "cuda" and input.dtype in _RS_DTYPES and output.dtype == input.dtype and input.is_contiguous()
            and output.is_contiguous() and block_bytes % 16 == 0 and input.data_ptr() % 16 == 0 and output.data_ptr() % 16 == 0
            and output.numel() * output.element_size() >= block_bytes):
        _lib.check(_lib.lib().tdist_ring_reduce(input.data_ptr(), output.data_ptr(), block_bytes, num_splits, begin_idx % num_splits,
                                                _RS_DTYPES[input.dtype], _stream_ptr(input.device)), "tdist_ring_reduce")
        launch_count += 1
        return output
    blocks = input.view(num_splits, M, *input.shape[1:])
    order = [(begin_idx + i) % num_splits for i in range(num_splits)]
    acc_dtype = torch.float32 if input.dtype in (torch.bfloat16, torch.float16) else input.dtype
    output.copy_(blocks[order].to(acc_dtype).sum(dim=0).to(output.dtype))
    return output


# ---------------------------------------------------------------------------- reference names kept for source compatibility
inter_node_allgather = cp_engine_producer_all_gather_intra_node   # reference allgather.py:470-624: one level on NVSwitch


def reduce_scatter_multi_node(input: torch.Tensor, ctx: ReduceScatter2DContext, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """reference reduce_scatter.py:766-783 (per-node scatter, then a cross-node ring): a single node here."""
    return reduce_scatter_2d_op(input, ctx, out=out)


def reduce_scatter_ring_push_1d_intra_node_kernel(input: torch.Tensor, ctx: ReduceScatter2DContext,
                                                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """reference reduce_scatter.py:344-426 (PCIe ring with SM copies). NVSwitch needs no ring: full-mesh push."""
    return reduce_scatter_2d_op(input, ctx, out=out)


reduce_scatter_ring_push_1d_intra_node_ce = reduce_scatter_ring_push_1d_intra_node_kernel  # reference :289-341
reduce_scatter_ring_push_1d_intra_node_sm = reduce_scatter_ring_push_1d_intra_node_kernel


def copy_continuous(src: torch.Tensor, dst: torch.Tensor, stream=None) -> torch.Tensor:
    """Contiguous device copy with this library's vector copy kernel (reference reduce_scatter.py:228-269
    ``copy_continuous_kernel``); ``dst`` may be a peer mapping."""
    if src.device.type != "cuda":
        dst.copy_(src)
        return dst
    n = src.numel() * src.element_size()
    if n % 16 or src.data_ptr() % 16 or dst.data_ptr() % 16 or not src.is_contiguous() or not dst.is_contiguous():
        dst.copy_(src)
        return dst
    _lib.check(_lib.lib().tdist_p2p_copy(src.data_ptr(), dst.data_ptr(), n, 0, min(64, max(1, n // 65536)), 512, 0,
                                         _status_ptr(), default_timeout_ns(), _stream_ptr(src.device, stream)), "tdist_p2p_copy")
    return dst


def add_continuous(lhs: torch.Tensor, rhs: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out = lhs + rhs`` with fp32 accumulation (reference reduce_scatter.py:186-225 ``add_continuous_kernel``): the
    two-source case of :func:`ring_reduce`."""
    stacked = torch.stack([lhs.reshape(-1, lhs.shape[-1]), rhs.reshape(-1, rhs.shape[-1])]).reshape(-1, lhs.shape[-1])
    o = out if out is not None else torch.empty_like(lhs)
    return ring_reduce(stacked, o.view(-1, lhs.shape[-1]), 0, 2).view_as(lhs)


def barrier_all_intra_node_non_atomic(local_world_size: int = 0, rank: int = 0, num_ranks: int = 0, symm_flags=None, target_value: int = 0,
                                      stream=None) -> None:
    """reference common_ops.py:104-159 (monotonic target values written to peers, then an acquire spin): exactly the
    protocol of the barrier kernel here, which keeps its own flags and target."""
    barrier_all_on_stream(stream)


barrier_all_intra_node_non_atomic_block = barrier_all_intra_node_non_atomic
# reference common_ops.py:88-101: CAS 0 -> 1 on the peers, then 1 -> 0 on the own flags. The monotonic barrier needs no
# reset phase and works over links without native atomics, so both names run it.
barrier_all_intra_node_atomic_cas_block = barrier_all_intra_node_non_atomic
