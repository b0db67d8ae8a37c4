"""Tensor-parallel GEMM ops backed by the tcgen05 kernel family in ``csrc/kernels/gemm_sm100.cu``.

Public surface (argument conventions of the reference):

* ``gemm_persistent(a[M,K], b[N,K]) -> [M,N]`` — plain GEMM
  (reference python/triton_dist/kernels/nvidia/allgather_gemm.py:978-1064).
* ``create_ag_gemm_intra_node_context`` / ``ag_gemm_intra_node(a[M/ws,K], b[N/ws,K], ctx) -> [M,N/ws]``
  (reference allgather_gemm.py:785-882).
* ``create_gemm_rs_context`` / ``gemm_rs(a[M,K/ws], b[N,K/ws], ctx) -> [M/ws,N]``
  (reference python/triton_dist/kernels/nvidia/gemm_reduce_scatter.py:77-87,524-538).

CUDA tensors run the fused sm_100a kernel (one launch per call: the gather / scatter happens
inside it over peer memory). CPU tensors run a torch + ``torch.distributed`` restatement that
serves as the oracle and as the gloo plumbing path.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib
from ..utils.profile import nvtx_range
from ..runtime import SymmTensor, counters_clean, default_timeout_ns, global_status, symm_heap

BLOCK_M = 128
BLOCK_N = 256
BLOCK_M_TILE = BLOCK_M  # module constants under names the keyword arguments below do not shadow
BLOCK_N_TILE = BLOCK_N

_DTYPES = {torch.bfloat16: _lib.DT_BF16, torch.float16: _lib.DT_F16}

# number of native launches since import (bench.py reports it)
launch_count = 0
# tiling choice handed to the kernel: -1 = automatic, 0 = one CTA per 128x256 tile,
# 1 = CTA pair (cta_group::2) per 256x256 tile, 2 = CTA pair per 256x512 tile; a context's `cta_pair` >= 0 overrides it
CTA_PAIR = int(os.environ.get("TDIST_GEMM_CTA_PAIR", "-1"))
# AG-GEMM pushers and multimem.st, when the heap has a multicast alias (TDIST_NVLS=1): 0 = never (default: on
# 8 x B200 the multicast pusher measured 1.18 ms against 0.98 ms for the unicast one on m8192 n49152 k12288),
# 1 = from 4 ranks up, 2 = always
AG_NVLS = int(os.environ.get("TDIST_AG_GEMM_NVLS", "0"))
# 1: the pushers of the fused AG-GEMM send each 128-row block as parallel row slices, so the first blocks land sooner.
# Off by default: with eight slices a pusher moved 24 GB/s instead of 36-38 (a flag hand-off per 400 KB), which costs
# more than the earlier first arrival gains now that the first round of tiles is split instead.
AG_PUSH_SLICES = int(os.environ.get("TDIST_AG_PUSH_SLICES", "0"))
GROUP_M = int(os.environ.get("TDIST_GEMM_GROUP_M", "0"))  # row-tiles per raster group, 0 = kernel default
TRACE = None  # optional int64[2048] device tensor: every launch writes its timeline there (layout: TdistGemmArgs.trace)


def _cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def _check_operands(a: torch.Tensor, b: torch.Tensor) -> None:
    if a.dtype != b.dtype or a.dtype not in _DTYPES:
        raise TypeError(f"GEMM operands must both be bf16 or fp16, got {a.dtype} and {b.dtype}")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise ValueError(f"expected a[M,K] and b[N,K], got {tuple(a.shape)} and {tuple(b.shape)}")
    if not a.is_contiguous() or not b.is_contiguous():
        raise ValueError("GEMM operands must be contiguous (K innermost)")
    if a.shape[1] % 8 or b.shape[0] % 8:
        raise ValueError("K and N must be multiples of 8")


def _base_args(a, b, world, rank, mode, stream=None, cta_pair: int = -1) -> "_lib.GemmArgs":
    g = _lib.GemmArgs()
    g.a = a.data_ptr()
    g.b = b.data_ptr()
    g.n = b.shape[0]
    g.k = a.shape[1]
    g.world = world
    g.rank = rank
    g.mode = mode
    g.dtype = _DTYPES[a.dtype]
    st = global_status()
    g.status = st.device_ptr if st is not None else None
    g.timeout_ns = default_timeout_ns()
    g.cta_pair = cta_pair if cta_pair >= 0 else CTA_PAIR
    g.group_m = GROUP_M
    if TRACE is not None:
        g.trace = TRACE.data_ptr()
    g.stream = (stream or torch.cuda.current_stream(a.device)).cuda_stream
    return g


def _launch(g: "_lib.GemmArgs") -> None:
    global launch_count
    _lib.check(_lib.lib().tdist_gemm_run(C.byref(g)), "tdist_gemm_run")
    launch_count += 1


# ---------------------------------------------------------------------------- plain GEMM
@nvtx_range("tdist.gemm_persistent")
def gemm_persistent(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
                    num_sms: int = 0) -> torch.Tensor:
    """``a[M,K] @ b[N,K].T`` with fp32 accumulation; output dtype = input dtype."""
    if a.device.type != "cuda":
        return (a.float() @ b.float().t()).to(a.dtype)
    _check_operands(a, b)
    M, N = a.shape[0], b.shape[0]
    c = out if out is not None else torch.empty((M, N), dtype=a.dtype, device=a.device)
    g = _base_args(a, b, 1, 0, _lib.GEMM_PLAIN)
    g.c = c.data_ptr()
    g.m_per_rank = M
    g.epoch = 1
    g.num_sms = num_sms
    _launch(g)
    return c


gemm_non_persistent = gemm_persistent  # one kernel family covers both reference variants


# ---------------------------------------------------------------------------- AllGather-GEMM
@dataclass
class AllGatherGEMMTensorParallelContext:
    """State of a column-parallel AG-GEMM: a double-buffered gather workspace and per-block
    arrival flags in symmetric memory, plus the call counter whose value the flags carry.

    ``workspace`` is ``[2, world * max_m_per_rank * K]`` elements; call ``e`` uses half ``e & 1``
    laid out as ``[world, m_per_rank, K]``. Two halves are enough: a rank can only start call
    ``e + 2`` after every peer has pushed call ``e + 1``, which each peer does after finishing
    its own call ``e``.
    """

    rank: int
    world: int
    max_m_per_rank: int
    k: int
    dtype: torch.dtype
    group: object = None
    workspace: Optional[SymmTensor] = None
    flags: Optional[SymmTensor] = None
    push_count: Optional[torch.Tensor] = None   # local slice-arrival counters of the pushers, one per (hop, block)
    epoch: int = 0
    num_comm_sms: int = 0   # 0 = sized per call from the bytes to push and the expected GEMM time
    num_sms: int = 0
    cta_pair: int = -1      # >= 0 overrides the module-wide tiling choice for this context
    for_correctness: bool = False
    debug_delay_ns: int = 0
    trace: Optional[torch.Tensor] = None  # int64[2048] timeline buffer, filled by the kernel when set


def create_ag_gemm_intra_node_context(tensor_A: torch.Tensor, tensor_B: torch.Tensor, rank: int, num_ranks: int,
                                      max_M: int = 2 ** 14, max_blocks: int = 65536, BLOCK_M: int = 128,
                                      BLOCK_N: int = 256, BLOCK_K: int = 64, stages: int = 4,
                                      for_correctness: bool = False, ag_stream=None, gemm_stream=None,
                                      serial: bool = False, autotune: bool = False, heap=None, group=None,
                                      num_comm_sms: int = 0) -> AllGatherGEMMTensorParallelContext:
    """Allocate the symmetric state for ``ag_gemm_intra_node``. ``max_M`` is the largest gathered
    row count. Tile shape, stage and stream arguments are accepted for source compatibility; the
    sm_100a kernel has one tuned configuration and needs no side streams."""
    K = tensor_A.shape[1]
    max_mpr = _cdiv(max_M, num_ranks)
    ctx = AllGatherGEMMTensorParallelContext(rank=rank, world=num_ranks, max_m_per_rank=max_mpr, k=K,
                                             dtype=tensor_A.dtype, group=group, for_correctness=for_correctness,
                                             num_comm_sms=num_comm_sms)
    if for_correctness:
        ctx.debug_delay_ns = 200_000
    if tensor_A.device.type == "cuda" and num_ranks > 1:
        heap = heap or symm_heap(group)
        ctx.workspace = heap.empty((2, num_ranks * max_mpr * K), tensor_A.dtype)
        ctx.flags = heap.zeros((2, num_ranks * _cdiv(max_mpr, BLOCK_M_TILE)), torch.int32)
        ctx.push_count = torch.zeros(num_ranks * _cdiv(max_mpr, BLOCK_M_TILE), dtype=torch.int32, device=tensor_A.device)
    return ctx



@nvtx_range("tdist.ag_gemm_intra_node")
def ag_gemm_intra_node(a: torch.Tensor, b: torch.Tensor, ctx: Optional[AllGatherGEMMTensorParallelContext] = None,
                       rank: Optional[int] = None, num_ranks: Optional[int] = None, persistent: bool = True,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``allgather(a) @ b.T``: ``a`` is this rank's ``[M/ws, K]`` row shard, ``b`` this rank's
    ``[N/ws, K]`` weight shard; returns ``[M, N/ws]``."""
    if ctx is None:
        if rank is None or num_ranks is None:
            raise ValueError("ag_gemm_intra_node needs a context or rank and num_ranks")
        ctx = create_ag_gemm_intra_node_context(a, b, rank, num_ranks)
    mpr, K = a.shape
    N = b.shape[0]
    if a.device.type != "cuda":
        return _ag_gemm_cpu(a, b, ctx)
    _check_operands(a, b)
    if mpr > ctx.max_m_per_rank or K != ctx.k:
        raise ValueError(f"shard {tuple(a.shape)} exceeds the context (max rows {ctx.max_m_per_rank}, K {ctx.k})")
    c = out if out is not None else torch.empty((ctx.world * mpr, N), dtype=a.dtype, device=a.device)
    g = _base_args(a, b, ctx.world, ctx.rank, _lib.GEMM_AG, cta_pair=ctx.cta_pair)
    g.c = c.data_ptr()
    g.m_per_rank = mpr
    ctx.epoch += 1
    g.epoch = ctx.epoch
    g.num_sms = ctx.num_sms
    g.num_comm_sms = ctx.num_comm_sms  # 0 = the launcher sizes it from the bytes to push and the GEMM's length
    g.debug_delay_ns = ctx.debug_delay_ns
    if ctx.trace is not None:
        g.trace = ctx.trace.data_ptr()
    if ctx.world > 1:
        half = ctx.epoch & 1
        g.a_ws = ctx.workspace.local[half].data_ptr()
        g.a_ws_peer = ctx.workspace.half_ptr_arrays()[half]
        g.flags = ctx.flags.local[half].data_ptr()
        g.flags_peer = ctx.flags.half_ptr_arrays()[half]
        if ctx.push_count is not None and AG_PUSH_SLICES:
            counters_clean(ctx.push_count)
            g.push_count = ctx.push_count.data_ptr()
        if ctx.workspace.mc is not None and (AG_NVLS == 2 or (AG_NVLS == 1 and ctx.world >= 4)):
            g.a_ws_mc = ctx.workspace.mc[half].data_ptr()   # the pushers multicast through the switch
    _launch(g)
    return c


def _ag_gemm_cpu(a, b, ctx):
    if ctx.world > 1:
        full = torch.empty((ctx.world * a.shape[0], a.shape[1]), dtype=a.dtype)
        dist.all_gather_into_tensor(full, a.contiguous(), group=ctx.group)
    else:
        full = a
    acc = torch.float32 if a.dtype in (torch.bfloat16, torch.float16) else a.dtype
    return (full.to(acc) @ b.to(acc).t()).to(a.dtype)


# ---------------------------------------------------------------------------- GEMM-ReduceScatter
@dataclass
class GEMMReduceScatterTensorParallelContext:
    """State of a row-parallel GEMM-RS: double-buffered staging ``[2, world * max_m_per_rank * N]``
    (half ``e & 1`` viewed as ``[src, m_per_rank, N]``) that the peers' epilogues store into, and
    per-(tile, source) arrival flags."""

    rank: int
    world: int
    max_m_per_rank: int
    n: int
    dtype: torch.dtype
    group: object = None
    staging: Optional[SymmTensor] = None
    flags: Optional[SymmTensor] = None
    epoch: int = 0
    num_sms: int = 0
    cta_pair: int = -1      # >= 0 overrides the module-wide tiling choice for this context


def create_gemm_rs_context(max_M: int, N: int, rank: int, world_size: int, local_world_size: Optional[int] = None,
                           output_dtype: torch.dtype = torch.bfloat16, rs_stream=None, BLOCK_M: int = 128,
                           BLOCK_N: int = 256, BLOCK_K: int = 64, GROUP_M: int = 8, stages: int = 4, heap=None,
                           group=None, device=None) -> GEMMReduceScatterTensorParallelContext:
    """Allocate the symmetric state for ``gemm_rs``; ``max_M`` is the largest un-scattered row
    count. Tile / stream arguments are accepted for source compatibility."""
    max_mpr = _cdiv(max_M, world_size)
    ctx = GEMMReduceScatterTensorParallelContext(rank=rank, world=world_size, max_m_per_rank=max_mpr, n=N,
                                                 dtype=output_dtype, group=group)
    on_cuda = (device is not None and torch.device(device).type == "cuda") or (device is None and torch.cuda.is_available())
    if on_cuda:
        heap = heap or symm_heap(group)
        ctx.staging = heap.empty((2, world_size * max_mpr * N), output_dtype)
        # one flag per (128-row block, 256-column tile, source); +1 block: a CTA pair may own a padding block
        tiles = (_cdiv(max_mpr, BLOCK_M_TILE) + 1) * _cdiv(N, BLOCK_N_TILE)
        ctx.flags = heap.zeros((2, tiles * world_size), torch.int32)
    return ctx



@nvtx_range("tdist.gemm_rs")
def gemm_rs(a: torch.Tensor, b: torch.Tensor, ctx: GEMMReduceScatterTensorParallelContext, persistent: bool = True,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``reduce_scatter_rows(a @ b.T)``: ``a`` is ``[M, K/ws]``, ``b`` is ``[N, K/ws]``; returns this
    rank's ``[M/ws, N]`` rows of the sum over ranks (fp32 reduction)."""
    M, _ = a.shape
    N = b.shape[0]
    if M % ctx.world:
        raise ValueError(f"M={M} must be divisible by the world size {ctx.world}")
    mpr = M // ctx.world
    if a.device.type != "cuda":
        return _gemm_rs_cpu(a, b, ctx)
    _check_operands(a, b)
    if mpr > ctx.max_m_per_rank or N != ctx.n:
        raise ValueError(f"problem [{M},{N}] exceeds the context (max rows/rank {ctx.max_m_per_rank}, N {ctx.n})")
    o = out if out is not None else torch.empty((mpr, N), dtype=a.dtype, device=a.device)
    if ctx.world == 1:
        return gemm_persistent(a, b, out=o, num_sms=ctx.num_sms)  # nothing to scatter or reduce: skip the staging pass
    g = _base_args(a, b, ctx.world, ctx.rank, _lib.GEMM_RS, cta_pair=ctx.cta_pair)
    g.m_per_rank = mpr
    ctx.epoch += 1
    g.epoch = ctx.epoch
    g.num_sms = ctx.num_sms
    half = ctx.epoch & 1
    g.c_stage_peer = ctx.staging.half_ptr_arrays()[half]
    g.flags = ctx.flags.local[half].data_ptr()
    g.flags_peer = ctx.flags.half_ptr_arrays()[half]
    g.rs_out = o.data_ptr()
    _launch(g)
    return o


def _gemm_rs_cpu(a, b, ctx):
    acc = torch.float32 if a.dtype in (torch.bfloat16, torch.float16) else a.dtype
    partial = a.to(acc) @ b.to(acc).t()
    if ctx.world == 1:
        return partial.to(a.dtype)
    out = torch.empty((partial.shape[0] // ctx.world, partial.shape[1]), dtype=acc)
    # gloo has no reduce_scatter: all_reduce and slice
    dist.all_reduce(partial, group=ctx.group)
    out.copy_(partial[ctx.rank * out.shape[0]:(ctx.rank + 1) * out.shape[0]])
    return out.to(a.dtype)


# ---------------------------------------------------------------------------- reference names kept for source compatibility
def create_ag_gemm_inter_node_context(tensor_A, tensor_B, rank, num_ranks, num_local_ranks: int = 8, max_M: int = 2 ** 14,
                                      **kw) -> AllGatherGEMMTensorParallelContext:
    """The reference's multi-node constructor (kernels/nvidia/allgather_gemm.py:885-935). One NVSwitch node is one
    level, so this is the intra-node context; more than one node is refused rather than silently mis-served."""
    if num_ranks > num_local_ranks:
        raise NotImplementedError("multi-node AG-GEMM is not built: one NVSwitch node (up to 8 ranks) is the target")
    return create_ag_gemm_intra_node_context(tensor_A, tensor_B, rank, num_ranks, max_M=max_M, **kw)


ag_gemm_inter_node = ag_gemm_intra_node  # reference allgather_gemm.py:938-975, same single-level kernel here


def padded_to_BLOCK_M(x: torch.Tensor, world_size: int, BLOCK_SIZE_M: int = BLOCK_M) -> torch.Tensor:
    """Pad every rank's row block of ``x [M, K]`` to a multiple of ``BLOCK_SIZE_M`` rows (reference
    gemm_reduce_scatter.py:468-479). The sm_100a kernels take ragged blocks (TMA clips them), so nothing here
    needs the padding; kept for callers that build padded layouts."""
    M = x.shape[0]
    mpr = M // world_size
    pad = (mpr + BLOCK_SIZE_M - 1) // BLOCK_SIZE_M * BLOCK_SIZE_M
    if pad == mpr:
        return x
    out = x.new_zeros((world_size, pad) + tuple(x.shape[1:]))
    out[:, :mpr].copy_(x.view(world_size, mpr, *x.shape[1:]))
    return out.view(world_size * pad, *x.shape[1:])


def gemm_rs_op(a: torch.Tensor, b: torch.Tensor, ctx: GEMMReduceScatterTensorParallelContext, persistent: bool = True,
               fuse_scatter: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """reference gemm_reduce_scatter.py:482-521; the scatter is always fused into the GEMM epilogue here."""
    return gemm_rs(a, b, ctx, persistent=persistent, out=out)


def local_copy_and_barrier_all(local_data: torch.Tensor, ctx: AllGatherGEMMTensorParallelContext) -> None:
    """reference allgather_gemm.py:99-114: stage this rank's shard in its own workspace slot and barrier. The fused
    kernel reads the own shard in place and orders calls by number, so this is only needed by code that drives
    the copy-engine producer (``cp_engine_producer_all_gather_intra_node``) against ``ctx.workspace`` itself."""
    from .collectives import barrier_all_on_stream
    if ctx.workspace is not None:
        mpr, K = local_data.shape
        ws = ctx.workspace.local[(ctx.epoch + 1) & 1][: ctx.world * mpr * K].view(ctx.world, mpr, K)
        ws[ctx.rank].copy_(local_data)
        barrier_all_on_stream()
