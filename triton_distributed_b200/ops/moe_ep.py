"""Expert-parallel MoE dispatch / combine: one launch each, routing and bookkeeping on the device.

``ep_dispatch`` sends every token to the ranks that own its ``topk`` experts and ``ep_combine`` brings the experts'
outputs back and sums them per token. They play the role of the reference's ``kernel_dispatch_token`` /
``kernel_combine_token`` / ``kernel_get_ag_splits_and_recv_offset`` / ``kernel_bincount``
(reference python/triton_dist/kernels/nvidia/ep_a2a.py:35-321) and of its ``EPAll2AllLayer``
(layers/nvidia/ep_a2a_layer.py:165-240), and of the quantising low-latency pair of tutorial 04
(tutorials/04-deepseek-infer-all2all.py:150-201).

Two receive layouts (see ``csrc/kernels/moe_ep.cu``):

* ``compact=False``: source ``s`` owns rows ``[s*max_m, (s+1)*max_m)`` of every receiver, sorted by local expert;
  no exchange precedes the rows (lowest latency).
* ``compact=True``: rows grouped by (local expert, source rank) back to back, each expert's group starting on a
  multiple of ``align`` rows; with ``align=128`` the receive buffer is directly the A operand of the grouped GEMM
  (``block_expert`` / ``num_blocks`` say which expert each 128-row block belongs to).

The expert outputs that ``ep_combine`` reads must sit in symmetric memory: ``expert_out_buffer(ctx)`` hands out the
buffer of the call in flight, row ``i`` of which answers row ``i`` of the receive buffer. Nothing here synchronises
with the host: counts (``num_recv``, ``recv_splits``, ...) are device tensors.

CUDA tensors run the kernels; CPU tensors (gloo ranks) run a torch.distributed restatement of the same layouts.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import _lib
from ..runtime import SymmTensor, default_timeout_ns, global_status, symm_heap
from ..utils.profile import nvtx_range
from . import moe_utils

launch_count = 0
ROUTE_IN_PLACE_MAX = 8192   # TDIST_MOE_ROUTE_IN_PLACE_MAX of csrc/include/tdist.h


@dataclass
class EPContext:
    max_tokens: int
    hidden: int
    topk: int
    num_experts: int
    rank: int
    world: int
    quant: bool
    compact: bool
    align: int
    max_m: int                                  # slots: rows per source slot; compact: capacity in rows
    rows: int                                   # rows of the receive / expert-output buffers
    group: object = None
    recv_buf: Optional[SymmTensor] = None       # [2, rows, hidden] fp8 (quant) or bf16
    scale_buf: Optional[SymmTensor] = None      # [2, rows, hidden / 128] fp32 (quant)
    counts_buf: Optional[SymmTensor] = None     # [2, world * num_experts] int32
    sig: Optional[SymmTensor] = None            # int64 [2 * MAX_RANKS] dispatch flags
    out_buf: Optional[SymmTensor] = None        # [2, rows, hidden] bf16 expert outputs
    comb_sig: Optional[SymmTensor] = None       # int64 [MAX_RANKS] combine flags
    counters: Optional[torch.Tensor] = None
    pair_row: Optional[torch.Tensor] = None     # int32 [max_tokens * topk]
    send_splits: Optional[torch.Tensor] = None  # int32 [num_experts]
    recv_splits: Optional[torch.Tensor] = None  # int32 [world, experts_per_rank]
    recv_offset: Optional[torch.Tensor] = None  # int32 [experts_per_rank, world]
    num_recv: Optional[torch.Tensor] = None     # int32 [1]
    block_expert: Optional[torch.Tensor] = None  # int32 [rows / align]
    num_blocks: Optional[torch.Tensor] = None   # int32 [1]
    call_count: int = 0
    combine_count: int = 0
    ntok: int = 0
    topk_ids: Optional[torch.Tensor] = None
    topk_weights: Optional[torch.Tensor] = None
    num_ctas: int = 0

    @property
    def experts_per_rank(self) -> int:
        return self.num_experts // self.world


def create_ep_context(max_tokens: int, hidden: int, topk: int, num_experts: int, rank: int, world_size: int,
                      quant: bool = False, compact: bool = True, align: int = 1, capacity: Optional[int] = None,
                      heap=None, group=None, device=None) -> EPContext:
    """``max_tokens`` = most tokens one rank dispatches per call. ``capacity`` (compact layout) = rows a rank can
    receive, default the worst case ``world * max_tokens * topk`` (plus the alignment padding)."""
    if num_experts % world_size:
        raise ValueError("the expert count must be a multiple of the world size")
    epr = num_experts // world_size
    max_m = max_tokens * topk
    if compact:
        rows = capacity if capacity is not None else world_size * max_m + epr * (align - 1)
        rows = (rows + align - 1) // align * align
        slot_rows = rows
    else:
        rows, slot_rows = world_size * max_m, max_m
    ctx = EPContext(max_tokens, hidden, topk, num_experts, rank, world_size, quant, compact, max(1, align), slot_rows, rows,
                    group=group)
    on_cuda = (device is not None and torch.device(device).type == "cuda") or (device is None and torch.cuda.is_available())
    if on_cuda:
        heap = heap or symm_heap(group)
        ctx.recv_buf = heap.empty((2, rows, hidden), torch.float8_e4m3fn if quant else torch.bfloat16)
        if quant:
            ctx.scale_buf = heap.empty((2, rows, hidden // 128), torch.float32)
        ctx.counts_buf = heap.zeros((2, world_size * num_experts), torch.int32)
        ctx.sig = heap.zeros((2 * _lib.MAX_RANKS,), torch.int64)
        ctx.out_buf = heap.empty((2, rows, hidden), torch.bfloat16)
        ctx.comb_sig = heap.zeros((_lib.MAX_RANKS,), torch.int64)
        dev = ctx.sig.local.device
        ctx.counters = torch.zeros(2, dtype=torch.int32, device=dev)
        ctx.pair_row = torch.full((max_m,), -1, dtype=torch.int32, device=dev)
        ctx.send_splits = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        ctx.recv_splits = torch.zeros((world_size, epr), dtype=torch.int32, device=dev)
        ctx.recv_offset = torch.zeros((epr, world_size), dtype=torch.int32, device=dev)
        ctx.num_recv = torch.zeros(1, dtype=torch.int32, device=dev)
        ctx.block_expert = torch.zeros(max(1, rows // max(1, align)), dtype=torch.int32, device=dev)
        ctx.num_blocks = torch.zeros(1, dtype=torch.int32, device=dev)
    return ctx


@nvtx_range("tdist.ep_dispatch")
def ep_dispatch(ctx: EPContext, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: Optional[torch.Tensor] = None,
                phase: int = 7, stream=None):
    """Send the rows of ``x`` bf16 ``[T, hidden]`` to the ranks owning the experts in ``topk_ids`` int32 ``[T, topk]``.

    Returns ``(recv, recv_scale, recv_splits, num_recv)``: views of this call's receive buffer ``[rows, hidden]``
    (fp8 with ``recv_scale`` fp32 ``[rows, hidden/128]`` when the context quantises, else bf16 and ``None``),
    ``recv_splits`` int32 ``[world, experts_per_rank]`` and ``num_recv`` int32 ``[1]``, all on the device. The views are
    valid for work enqueued before the next dispatch on this context.

    ``phase`` (for running emulated ranks one after the other): bit 0 publishes this rank's per-expert counts
    (compact layout only), bit 1 routes, sends and raises the flags, bit 2 waits for every source."""
    global launch_count
    T = x.shape[0]
    if T > ctx.max_tokens:
        raise ValueError("more tokens than the context was built for")
    if x.device.type != "cuda":
        return _ep_dispatch_cpu(ctx, x, topk_ids, topk_weights)
    if x.dtype != torch.bfloat16 or not x.is_contiguous() or x.shape[1] != ctx.hidden:
        raise ValueError("x must be contiguous bf16 [T, hidden]")
    first = bool(phase & 1) if ctx.compact else bool(phase & 2)   # the first launch of a call advances the call number
    if first:
        ctx.call_count += 1
        ctx.topk_ids = topk_ids.to(torch.int32).contiguous()
        ctx.topk_weights = None if topk_weights is None else topk_weights.to(torch.float32).contiguous()
        ctx.ntok = T
    half = ctx.call_count & 1
    a = _lib.MoeDispatchArgs()
    a.x, a.topk_ids = x.data_ptr(), ctx.topk_ids.data_ptr()
    routed = None
    if T * ctx.topk > ROUTE_IN_PLACE_MAX:
        routed = moe_utils.route(ctx.topk_ids, ctx.num_experts)     # large batches: routing as a launch of its own
        a.slot_of, a.cumsum = routed.slot_of.data_ptr(), routed.cumsum.data_ptr()
    a.recv_peer = ctx.recv_buf.half_ptr_arrays()[half]
    if ctx.quant:
        a.scale_peer = ctx.scale_buf.half_ptr_arrays()[half]
    a.counts_peer = ctx.counts_buf.half_ptr_arrays()[half]
    a.sig_peer = ctx.sig.cached_ptr_array()
    a.counters = ctx.counters.data_ptr()
    a.pair_row, a.send_splits = ctx.pair_row.data_ptr(), ctx.send_splits.data_ptr()
    a.recv_splits, a.recv_offset = ctx.recv_splits.data_ptr(), ctx.recv_offset.data_ptr()
    a.num_recv = ctx.num_recv.data_ptr()
    if ctx.compact:
        a.block_expert, a.num_blocks = ctx.block_expert.data_ptr(), ctx.num_blocks.data_ptr()
    a.ntok, a.topk, a.hidden, a.num_experts = T, ctx.topk, ctx.hidden, ctx.num_experts
    a.world, a.rank = ctx.world, ctx.rank
    a.max_m, a.quant, a.compact, a.align = ctx.max_m, int(ctx.quant), int(ctx.compact), ctx.align
    a.phase, a.num_ctas, a.epoch = phase, ctx.num_ctas, ctx.call_count
    st = global_status()
    a.status = st.device_ptr if st is not None else None
    a.timeout_ns = default_timeout_ns()
    a.stream = (stream or torch.cuda.current_stream(x.device)).cuda_stream
    _lib.check(_lib.lib().tdist_moe_dispatch(C.byref(a)), "tdist_moe_dispatch")
    launch_count += 1
    return (ctx.recv_buf.local[half], ctx.scale_buf.local[half] if ctx.quant else None, ctx.recv_splits, ctx.num_recv)


def expert_out_buffer(ctx: EPContext) -> torch.Tensor:
    """The symmetric bf16 buffer ``[rows, hidden]`` the experts of the call in flight write their outputs into
    (row ``i`` answers row ``i`` of the receive buffer); ``ep_combine`` of the peers reads it in place."""
    if ctx.out_buf is None:
        raise ValueError("no symmetric buffers on this device")
    return ctx.out_buf.local[ctx.call_count & 1]


@nvtx_range("tdist.ep_combine")
def ep_combine(ctx: EPContext, expert_out: Optional[torch.Tensor] = None, weighted: bool = True,
               out: Optional[torch.Tensor] = None, phase: int = 3, stream=None) -> torch.Tensor:
    """``out[t] = sum_k w[t,k] * expert_out_of_owner(t,k)`` (plain sum when ``weighted`` is false or the dispatch got
    no weights), bf16 ``[T, hidden]``, fp32 accumulation. ``expert_out`` is the tensor returned by
    :func:`expert_out_buffer` (the default), or any bf16 ``[rows, hidden]`` tensor in the receive layout, which is
    then first copied into that buffer. ``phase``: bit 0 announces this rank's outputs, bit 1 waits and gathers."""
    global launch_count
    T = ctx.ntok
    if ctx.out_buf is None:
        return _ep_combine_cpu(ctx, expert_out, weighted)
    half = ctx.call_count & 1
    buf = ctx.out_buf.local[half]
    if expert_out is not None and expert_out.data_ptr() != buf.data_ptr() and (phase & 1):
        if expert_out.dtype != torch.bfloat16 or expert_out.shape[1] != ctx.hidden or expert_out.shape[0] > ctx.rows:
            raise ValueError("expert_out must be bf16 [rows, hidden] in the receive layout")
        buf[: expert_out.shape[0]].copy_(expert_out)
    if phase & 1:
        ctx.combine_count += 1
    o = out if out is not None else torch.empty((T, ctx.hidden), dtype=torch.bfloat16, device=buf.device)
    a = _lib.MoeCombineArgs()
    a.buf_peer = ctx.out_buf.half_ptr_arrays()[half]
    a.sig_peer = ctx.comb_sig.cached_ptr_array()
    a.topk_ids = ctx.topk_ids.data_ptr()
    a.topk_w = ctx.topk_weights.data_ptr() if (weighted and ctx.topk_weights is not None) else None
    a.pair_row, a.out = ctx.pair_row.data_ptr(), o.data_ptr()
    a.ntok, a.topk, a.hidden, a.epr = T, ctx.topk, ctx.hidden, ctx.experts_per_rank
    a.world, a.rank, a.phase, a.num_ctas, a.epoch = ctx.world, ctx.rank, phase, 0, ctx.combine_count
    st = global_status()
    a.status = st.device_ptr if st is not None else None
    a.timeout_ns = default_timeout_ns()
    a.stream = (stream or torch.cuda.current_stream(buf.device)).cuda_stream
    _lib.check(_lib.lib().tdist_moe_combine(C.byref(a)), "tdist_moe_combine")
    launch_count += 1
    return o


# ---------------------------------------------------------------------------- CPU restatement (gloo ranks)
def _gather(t: torch.Tensor, ctx: EPContext):
    if ctx.world == 1:
        return [t]
    outs = [torch.empty_like(t) for _ in range(ctx.world)]
    dist.all_gather(outs, t.contiguous(), group=ctx.group)
    return outs


def _ep_layout_cpu(ctx: EPContext, all_ids):
    """Row of every (source, pair) in every destination, per the layout rules of the kernel."""
    W, E, epr, K = ctx.world, ctx.num_experts, ctx.experts_per_rank, ctx.topk
    counts = torch.stack([torch.bincount(ids.reshape(-1).long().clamp(0, E), minlength=E + 1)[:E] for ids in all_ids])  # [W, E]
    rows = []
    al = ctx.align
    tot = counts.sum(0)
    padded = (tot + al - 1) // al * al
    for s in range(W):
        ids = all_ids[s].reshape(-1).long()
        ok = (ids >= 0) & (ids < E)
        r = moe_utils.route(all_ids[s].reshape(-1, K), E)
        within = r.slot_of.long() - r.cumsum.long()[ids.clamp(0, E - 1)]
        if ctx.compact:
            group_start = torch.zeros(E, dtype=torch.long)
            for d in range(W):
                seg = padded[d * epr:(d + 1) * epr]
                group_start[d * epr:(d + 1) * epr] = torch.cumsum(seg, 0) - seg
            base = group_start + counts[:s].sum(0)
            row = base[ids.clamp(0, E - 1)] + within
        else:
            first = r.cumsum.long()[(ids.clamp(0, E - 1) // epr) * epr]
            row = s * ctx.max_m + r.slot_of.long() - first
        rows.append(torch.where(ok, row, torch.full_like(row, -1)))
    return counts, rows


def _ep_dispatch_cpu(ctx: EPContext, x, topk_ids, topk_weights):
    ctx.call_count += 1
    ctx.topk_ids = topk_ids.to(torch.int32).contiguous()
    ctx.topk_weights = None if topk_weights is None else topk_weights.float().contiguous()
    ctx.ntok = x.shape[0]
    T, K, W, epr = ctx.max_tokens, ctx.topk, ctx.world, ctx.experts_per_rank
    pad_x = torch.zeros((T, ctx.hidden), dtype=torch.float32)
    pad_x[: x.shape[0]] = x.float()
    pad_ids = torch.full((T, K), -1, dtype=torch.int32)
    pad_ids[: x.shape[0]] = ctx.topk_ids
    all_x, all_ids = _gather(pad_x, ctx), _gather(pad_ids, ctx)
    counts, rows = _ep_layout_cpu(ctx, all_ids)
    recv = torch.zeros((ctx.rows, ctx.hidden), dtype=torch.float32)
    for s in range(W):
        ids = all_ids[s].reshape(-1).long()
        mine = (rows[s] >= 0) & (ids // epr == ctx.rank)
        recv[rows[s][mine]] = all_x[s][(torch.arange(T * K) // K)[mine]]
    ctx._cpu_rows = rows
    ctx.pair_row = rows[ctx.rank][: x.shape[0] * K].to(torch.int32)
    ctx.recv_splits = counts[:, ctx.rank * epr:(ctx.rank + 1) * epr].to(torch.int32).contiguous()
    ctx.num_recv = ctx.recv_splits.sum().reshape(1).to(torch.int32)
    scale = None
    if ctx.quant:
        from .all_to_all import quant_fp8_reference
        q, scale = quant_fp8_reference(recv.to(torch.bfloat16))
        return q, scale, ctx.recv_splits, ctx.num_recv
    return recv.to(torch.bfloat16), scale, ctx.recv_splits, ctx.num_recv


def _ep_combine_cpu(ctx: EPContext, expert_out, weighted):
    if expert_out is None:
        raise ValueError("on CPU the expert outputs are passed in")
    pad = torch.zeros((ctx.rows, ctx.hidden), dtype=torch.float32)
    pad[: expert_out.shape[0]] = expert_out.float()
    outs = _gather(pad, ctx)
    T, K, epr = ctx.ntok, ctx.topk, ctx.experts_per_rank
    ids = ctx.topk_ids.reshape(-1).long()
    row = ctx.pair_row.long()
    ok = row >= 0
    dest = (ids.clamp(min=0) // epr).clamp(max=ctx.world - 1)
    vals = torch.zeros((T * K, ctx.hidden), dtype=torch.float32)
    for d in range(ctx.world):
        sel = ok & (dest == d)
        vals[sel] = outs[d][row[sel]]
    if weighted and ctx.topk_weights is not None:
        vals = vals * ctx.topk_weights.reshape(-1, 1)
    return vals.view(T, K, -1).sum(1).to(torch.bfloat16)
