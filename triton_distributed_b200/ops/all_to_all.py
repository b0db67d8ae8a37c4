"""Low-latency MoE all-to-all (expert-parallel dispatch / combine).

Two levels:

* the reference's generic op — ``create_all_to_all_context`` / ``fast_all_to_all(ctx, send[ntok,hidden],
  send_split_cumsum[G+1], send_scale) -> (recv_splits[G], recv[ws*max_m, hidden], recv_scale)`` and
  ``all_to_all_post_process`` (reference kernels/nvidia/low_latency_all_to_all.py:125-270): rows
  already sorted by expert, source rank ``r`` lands in rows ``[r*max_m, r*max_m + count_r)``;
* a fused MoE pair ``moe_dispatch`` / ``moe_combine`` for the serving layout of the reference's
  tutorial 04 (tutorials/04-deepseek-infer-all2all.py:150-201): dispatch gathers rows by the routing
  permutation, quantises bf16 to fp8 e4m3 with one fp32 scale per 128 values on the fly and ships
  rows + scales + per-expert counts in one launch; combine ships the experts' bf16 outputs back and
  applies the top-k weights in the same launch.

CUDA tensors run ``csrc/kernels/a2a.cu``; CPU tensors run a torch.distributed restatement.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import _lib
from ..utils.profile import nvtx_range
from ..runtime import SymmTensor, default_timeout_ns, global_status, symm_heap
from . import moe_utils

launch_count = 0


@dataclass
class AllToAllContext:
    max_m: int
    hidden: int
    rank: int
    num_tot_experts: int
    WORLD_SIZE: int
    experts_per_rank: int
    dtype: torch.dtype
    scale_dtype: torch.dtype
    scale_cols: int = 1
    recv_buf: Optional[SymmTensor] = None        # [2, world*max_m, hidden]
    scale_recv_buf: Optional[SymmTensor] = None  # [2, world*max_m, scale_cols] fp32
    split_recv_buf: Optional[SymmTensor] = None  # [2, world*epr] int32
    signal_buf: Optional[SymmTensor] = None      # int64 [8]
    counters: Optional[torch.Tensor] = None
    call_count: int = 0
    ctas_per_peer: int = 0
    group: object = None


def create_all_to_all_context(max_m: int, hidden: int, rank: int, num_tot_experts: int, WORLD_SIZE: int,
                              experts_per_rank: int, dtype: torch.dtype = torch.bfloat16,
                              scale_dtype: torch.dtype = torch.float32, scale_cols: int = 1, heap=None, group=None,
                              device=None) -> AllToAllContext:
    """``max_m`` = most rows one rank sends in one call (tokens * topk). ``scale_cols`` = fp32 scales
    carried per row (1 in the reference's test, hidden/128 for block-scaled fp8)."""
    ctx = AllToAllContext(max_m, hidden, rank, num_tot_experts, WORLD_SIZE, experts_per_rank, dtype, scale_dtype,
                          scale_cols, group=group)
    on_cuda = (device is not None and torch.device(device).type == "cuda") or (device is None and torch.cuda.is_available())
    if on_cuda:
        heap = heap or symm_heap(group)
        ctx.recv_buf = heap.empty((2, WORLD_SIZE * max_m, hidden), dtype)
        ctx.scale_recv_buf = heap.empty((2, WORLD_SIZE * max_m, scale_cols), torch.float32)
        ctx.split_recv_buf = heap.zeros((2, WORLD_SIZE * experts_per_rank), torch.int32)
        ctx.signal_buf = heap.zeros((_lib.MAX_RANKS,), torch.int64)
        ctx.counters = torch.zeros(_lib.MAX_RANKS, dtype=torch.int32, device=ctx.signal_buf.local.device)
    return ctx


def _fill_common(a: "_lib.A2AArgs", ctx: AllToAllContext, half: int, phase: int, device, stream) -> None:
    a.recv_peer = ctx.recv_buf.half_ptr_arrays()[half]
    a.scale_peer = ctx.scale_recv_buf.half_ptr_arrays()[half]
    a.splits_peer = ctx.split_recv_buf.half_ptr_arrays()[half]
    a.sig_peer = ctx.signal_buf.cached_ptr_array()
    a.counters = ctx.counters.data_ptr()
    a.max_m, a.epr, a.world, a.rank = ctx.max_m, ctx.experts_per_rank, ctx.WORLD_SIZE, ctx.rank
    a.phase = phase
    a.ctas_per_peer = ctx.ctas_per_peer
    a.epoch = ctx.call_count
    st = global_status()
    a.status = st.device_ptr if st is not None else None
    a.timeout_ns = default_timeout_ns()
    a.stream = (stream or torch.cuda.current_stream(device)).cuda_stream


def _next_call(ctx: AllToAllContext, phase: int) -> int:
    """Advance the call counter (not for a receive-only half) and return the buffer parity."""
    if phase != 2:
        ctx.call_count += 1
    return ctx.call_count & 1


def _launch(a: "_lib.A2AArgs") -> None:
    global launch_count
    _lib.check(_lib.lib().tdist_a2a(C.byref(a)), "tdist_a2a")
    launch_count += 1


@nvtx_range("tdist.fast_all_to_all")
def fast_all_to_all(ctx: AllToAllContext, send_tensor: torch.Tensor, send_split_cumsum: torch.Tensor,
                    send_scale: Optional[torch.Tensor] = None, phase: int = 3, stream=None):
    """Rows ``[cumsum[e], cumsum[e+1])`` of ``send_tensor`` go to the rank owning expert ``e``.
    Returns views into this call's half of the receive buffers: ``(recv_splits[G] int32 laid out
    [source rank, local expert], recv[ws*max_m, hidden], recv_scale[ws*max_m, scale_cols] | None)``.
    The views are valid only for work enqueued before the next call on this context: a peer may start
    the call after next as soon as this rank's next call has pushed, and then overwrites this half.
    A destination that would get more than ``max_m`` rows from this rank receives ``max_m`` (its splits say so)
    and the status block records a bad argument, which ``check_status()`` raises."""
    ntok = send_tensor.shape[0]
    # one destination never gets more than max_m rows from one source; the sender as a whole may hold
    # up to world * max_m rows (the combine direction sends back everything it received)
    if ntok > ctx.WORLD_SIZE * ctx.max_m:
        raise ValueError(f"{ntok} rows exceed world * max_m = {ctx.WORLD_SIZE * ctx.max_m}")
    if send_tensor.device.type != "cuda":
        return _fast_all_to_all_cpu(ctx, send_tensor, send_split_cumsum, send_scale)
    if not send_tensor.is_contiguous() or send_tensor.shape[1] != ctx.hidden or send_tensor.dtype != ctx.dtype:
        raise ValueError("send_tensor must be contiguous [rows, hidden] of the context's dtype")
    half = _next_call(ctx, phase)
    a = _lib.A2AArgs()
    a.send = send_tensor.data_ptr()
    cums = send_split_cumsum if send_split_cumsum.dtype == torch.int32 else send_split_cumsum.to(torch.int32)
    a.counts = cums.data_ptr()
    scale = None
    if send_scale is not None:
        scale = send_scale.reshape(ntok, -1).to(torch.float32).contiguous()
        if scale.shape[1] != ctx.scale_cols:
            raise ValueError(f"send_scale has {scale.shape[1]} columns, context was built for {ctx.scale_cols}")
        a.send_scale = scale.data_ptr()
    a.row_bytes_in = a.row_bytes_out = ctx.hidden * send_tensor.element_size()
    a.scale_cols, a.hidden = ctx.scale_cols, ctx.hidden
    a.mode = _lib.A2A_DISPATCH
    _fill_common(a, ctx, half, phase, send_tensor.device, stream)
    _launch(a)
    return (ctx.split_recv_buf.local[half], ctx.recv_buf.local[half],
            ctx.scale_recv_buf.local[half] if send_scale is not None else None)


def all_to_all_post_process(ctx: AllToAllContext, input_splits: torch.Tensor, recv_buffer: torch.Tensor,
                            scale_buffer: Optional[torch.Tensor] = None):
    """Compact the per-source slots of a receive buffer into one contiguous tensor (host sync on
    the counts, like the reference)."""
    per_rank = input_splits.reshape(ctx.WORLD_SIZE, -1).sum(dim=1).tolist()
    data = torch.cat([recv_buffer[i * ctx.max_m: i * ctx.max_m + n] for i, n in enumerate(per_rank)])
    scale = None
    if scale_buffer is not None:
        scale = torch.cat([scale_buffer[i * ctx.max_m: i * ctx.max_m + n] for i, n in enumerate(per_rank)])
    return data, scale


def _fast_all_to_all_cpu(ctx, send, cumsum, scale):
    W, epr, mm = ctx.WORLD_SIZE, ctx.experts_per_rank, ctx.max_m
    pad = torch.zeros((W * mm, send.shape[1]), dtype=send.dtype)
    pad[: send.shape[0]] = send
    cums = cumsum.to(torch.int32)
    scol = ctx.scale_cols
    spad = torch.zeros((W * mm, scol), dtype=torch.float32)
    if scale is not None:
        spad[: send.shape[0]] = scale.reshape(send.shape[0], -1).float()
    if W > 1:
        all_rows = [torch.empty_like(pad) for _ in range(W)]
        all_cums = [torch.empty_like(cums) for _ in range(W)]
        all_scales = [torch.empty_like(spad) for _ in range(W)]
        dist.all_gather(all_rows, pad, group=ctx.group)
        dist.all_gather(all_cums, cums, group=ctx.group)
        dist.all_gather(all_scales, spad, group=ctx.group)
    else:
        all_rows, all_cums, all_scales = [pad], [cums], [spad]
    recv = torch.zeros((W * mm, send.shape[1]), dtype=send.dtype)
    rscale = torch.zeros((W * mm, scol), dtype=torch.float32)
    splits = torch.zeros(W * epr, dtype=torch.int32)
    for s in range(W):
        c = all_cums[s]
        lo, hi = int(c[ctx.rank * epr]), int(c[(ctx.rank + 1) * epr])
        recv[s * mm: s * mm + hi - lo] = all_rows[s][lo:hi]
        rscale[s * mm: s * mm + hi - lo] = all_scales[s][lo:hi]
        splits[s * epr:(s + 1) * epr] = c[ctx.rank * epr + 1:(ctx.rank + 1) * epr + 1] - c[ctx.rank * epr:(ctx.rank + 1) * epr]
    return splits, recv, (rscale if scale is not None else None)


# ---------------------------------------------------------------------------- fused MoE pair
@dataclass
class MoEDispatchContext:
    """State of the fused dispatch / combine pair for the serving layout: fp8 rows with hidden/128 scales out
    (per-source slots, routing done inside the dispatch kernel), bf16 expert outputs pulled back by the combine.
    ``ep`` is the underlying expert-parallel context (``ops/moe_ep.py``)."""

    ep: "object"
    num_experts: int
    topk: int
    hidden: int

    @property
    def max_m(self) -> int:
        return self.ep.max_m

    @property
    def ntok(self) -> int:
        return self.ep.ntok


def create_moe_dispatch_context(max_tokens: int, hidden: int, topk: int, num_experts: int, rank: int, world_size: int,
                                heap=None, group=None, device=None) -> MoEDispatchContext:
    from . import moe_ep
    ep = moe_ep.create_ep_context(max_tokens, hidden, topk, num_experts, rank, world_size, quant=True, compact=False,
                                  heap=heap, group=group, device=device)
    return MoEDispatchContext(ep, num_experts, topk, hidden)


@nvtx_range("tdist.moe_dispatch")
def moe_dispatch(ctx: MoEDispatchContext, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                 phase: int = 3, stream=None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Send every token to the ranks of its ``topk`` experts as fp8 e4m3 with per-128 fp32 scales: one launch that
    sorts the (token, k) pairs by expert, quantises each token once and stores it into every owner's slot.

    ``x`` bf16 ``[T, hidden]``, ``topk_ids`` int32 ``[T, topk]``. Returns views into the receive
    buffers: ``(recv_x fp8 [ws*max_m, hidden], recv_scale fp32 [ws*max_m, hidden/128], recv_splits
    int32 [ws, experts_per_rank])``; source ``s`` occupies rows ``[s*max_m, s*max_m + sum(splits[s]))``
    sorted by local expert. ``phase`` 1 = send only, 2 = wait only (emulated ranks), 3 = both."""
    from . import moe_ep
    rx, rs, splits, _ = moe_ep.ep_dispatch(ctx.ep, x, topk_ids, topk_weights, phase=(phase & 3) << 1, stream=stream)
    return rx, rs, splits


def moe_expert_out_buffer(ctx: MoEDispatchContext) -> torch.Tensor:
    """Where the experts of the call in flight write their bf16 outputs (``[ws*max_m, hidden]``, receive layout) for
    :func:`moe_combine` to read in place."""
    from . import moe_ep
    return moe_ep.expert_out_buffer(ctx.ep)


@nvtx_range("tdist.moe_combine")
def moe_combine(ctx: MoEDispatchContext, expert_out: Optional[torch.Tensor] = None, recv_splits: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, phase: int = 3, stream=None) -> torch.Tensor:
    """Bring the experts' outputs back to their source ranks and reduce over ``topk`` with the gate
    weights of the matching ``moe_dispatch``: every rank reads the rows of its tokens straight from the owners'
    buffers (peer loads) and sums them in fp32.

    ``expert_out`` bf16 ``[ws*max_m, hidden]`` in the receive layout of ``moe_dispatch`` (row i of
    the output corresponds to row i of ``recv_x``); pass :func:`moe_expert_out_buffer` (or nothing) when the
    experts wrote there, any other tensor is copied there first. Returns bf16 ``[T, hidden]``."""
    from . import moe_ep
    return moe_ep.ep_combine(ctx.ep, expert_out, weighted=True, out=out, phase=phase, stream=stream)


def dequant_fp8(x: torch.Tensor, scale: torch.Tensor, rows: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp8 e4m3 ``[R, hidden]`` with fp32 scales ``[R, hidden/128]`` -> bf16 ``[R, hidden]`` (into ``out`` when given)."""
    global launch_count
    R = x.shape[0] if rows is None else rows
    hidden = x.shape[1]
    if x.device.type != "cuda":
        return (x[:R].float().view(R, hidden // 128, 128) * scale[:R].float().unsqueeze(-1)).view(R, hidden).to(torch.bfloat16)
    if out is None:
        out = torch.empty((x.shape[0], hidden), dtype=torch.bfloat16, device=x.device)
    _lib.check(_lib.lib().tdist_dequant_fp8(x.data_ptr(), scale.data_ptr(), out.data_ptr(), R, hidden,
                                            torch.cuda.current_stream(x.device).cuda_stream), "tdist_dequant_fp8")
    launch_count += 1
    return out


def quant_fp8_reference(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Torch statement of the on-the-fly quantisation (oracle): per row, per 128 values,
    scale = amax / 448, q = x / scale rounded to e4m3."""
    R, H = x.shape
    g = x.float().view(R, H // 128, 128)
    scale = g.abs().amax(-1).clamp_min(1e-10) / 448.0
    q = (g / scale.unsqueeze(-1)).view(R, H).to(torch.float8_e4m3fn)
    return q, scale


# ---------------------------------------------------------------------------- helpers of the reference's EP layer
def get_ag_splits_and_recv_offset_for_dispatch(send_splits: torch.Tensor, world_size: int, experts_per_rank: int, group=None):
    """From this rank's per-expert send counts ``[num_experts]`` build what the dispatch needs (reference
    kernels/nvidia/ep_a2a.py:352-387): ``recv_splits [world, experts_per_rank]`` (rows each source sends to my experts),
    ``recv_offset [experts_per_rank, world]`` (exclusive prefix sum in (expert, source) order = where each (expert,
    source) group starts in the regrouped receive layout) and ``num_recv`` (rows I receive in total). A set-up
    collective (NCCL / gloo all-gather), not a hot path: the fused dispatch kernel carries the splits itself."""
    splits = send_splits.to(torch.int32).contiguous()
    if world_size > 1:
        gathered = torch.empty((world_size, splits.numel()), dtype=torch.int32, device=splits.device)
        dist.all_gather_into_tensor(gathered, splits, group=group)
        rank = dist.get_rank(group)
    else:
        gathered, rank = splits.view(1, -1), 0
    recv_splits = gathered[:, rank * experts_per_rank:(rank + 1) * experts_per_rank].contiguous()     # [src, e]
    by_expert = recv_splits.t().contiguous()                                                            # [e, src]
    flat = by_expert.reshape(-1).to(torch.int64)
    recv_offset = (torch.cumsum(flat, 0) - flat).view(experts_per_rank, world_size).to(torch.int32)
    return recv_splits, recv_offset, int(flat.sum())


def get_dispatch_send_reqs_for_target_node(token_node_idx: torch.Tensor, traget_node_id: int, index_type=torch.int32):
    """Contiguous ``[start, end)`` ranges of tokens bound for one node (reference ep_a2a.py:338-350; the spelling of the
    second argument is the reference's). With a single NVSwitch node every token's node is 0 and the answer is one range."""
    hit = (token_node_idx == traget_node_id).any(dim=-1) if token_node_idx.dim() > 1 else (token_node_idx == traget_node_id)
    idx = torch.nonzero(hit, as_tuple=False).flatten()
    if idx.numel() == 0:
        return torch.empty((0, 2), dtype=index_type, device=token_node_idx.device)
    breaks = torch.nonzero(idx[1:] != idx[:-1] + 1, as_tuple=False).flatten()
    starts = torch.cat([idx[:1], idx[breaks + 1]])
    ends = torch.cat([idx[breaks], idx[-1:]]) + 1
    return torch.stack([starts, ends], dim=1).to(index_type)
