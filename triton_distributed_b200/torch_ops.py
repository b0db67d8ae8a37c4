"""``torch.ops.tdist.*``: the op library registered with ``torch.library``.

Every op here is a thin registration over the functions in :mod:`triton_distributed_b200.ops`, with
the reference's argument shapes and layouts. Stateful ops (anything that owns symmetric buffers
and a call counter) take the *handle* of a context created on the Python side
(``register_context(ctx) -> int``), because a custom op's arguments must be tensors and plain
numbers. Each op has a fake (meta) implementation, so shapes and dtypes propagate under
``torch.compile`` / FakeTensor tracing without touching a GPU.

The reference exposes its CUDA helper op through a pybind registry (reference csrc/lib/registry.h:31-53,
op_pybind.cc:33-44) and its Triton ops as plain Python functions; here both kinds go through one
dispatcher namespace.

    import triton_distributed_b200.torch_ops as T
    h = T.register_context(G.create_ag_gemm_intra_node_context(a, w, rank, world))
    c = torch.ops.tdist.ag_gemm(a, w, h)
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from .ops import all_to_all as A
from .ops import collectives as CO
from .ops import flash_decode as FD
from .ops import gemm as G
from .ops import gemm_fp8 as F8
from .ops import moe_tp as MT
from .ops import moe_utils as MU

_CONTEXTS: Dict[int, object] = {}
_NEXT = [1]


def register_context(ctx) -> int:
    """Park a context object and return the integer handle the ``tdist`` ops take."""
    h = _NEXT[0]
    _NEXT[0] += 1
    _CONTEXTS[h] = ctx
    return h


def get_context(handle: int):
    return _CONTEXTS[handle]


def release_context(handle: int) -> None:
    _CONTEXTS.pop(handle, None)


_op = torch.library.custom_op


# ---------------------------------------------------------------------------- GEMM family
@_op("tdist::gemm", mutates_args=())
def gemm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a[M,K] @ b[N,K]^T"""
    return G.gemm_persistent(a, b)


@gemm.register_fake
def _(a, b):
    return a.new_empty((a.shape[0], b.shape[0]))


@_op("tdist::ag_gemm", mutates_args=())
def ag_gemm(a: torch.Tensor, b: torch.Tensor, ctx: int) -> torch.Tensor:
    """allgather(a[M/ws,K]) @ b[N/ws,K]^T -> [M, N/ws]"""
    return G.ag_gemm_intra_node(a, b, _CONTEXTS[ctx])


@ag_gemm.register_fake
def _(a, b, ctx):
    return a.new_empty((a.shape[0] * _CONTEXTS[ctx].world, b.shape[0]))


@_op("tdist::gemm_rs", mutates_args=())
def gemm_rs(a: torch.Tensor, b: torch.Tensor, ctx: int) -> torch.Tensor:
    """reduce_scatter_rows(a[M,K/ws] @ b[N,K/ws]^T) -> [M/ws, N]"""
    return G.gemm_rs(a, b, _CONTEXTS[ctx])


@gemm_rs.register_fake
def _(a, b, ctx):
    return a.new_empty((a.shape[0] // _CONTEXTS[ctx].world, b.shape[0]))


@_op("tdist::group_gemm", mutates_args=())
def group_gemm(a_sorted: torch.Tensor, b: torch.Tensor, expert_ids: torch.Tensor, num_blocks: torch.Tensor) -> torch.Tensor:
    """128-row block i of a_sorted times b[expert_ids[i]][N,K]^T"""
    return MT.group_gemm(a_sorted, b, expert_ids, num_blocks)


@group_gemm.register_fake
def _(a_sorted, b, expert_ids, num_blocks):
    return a_sorted.new_empty((a_sorted.shape[0], b.shape[1]))


@_op("tdist::gemm_fp8", mutates_args=())
def gemm_fp8(a: torch.Tensor, sa: torch.Tensor, b: torch.Tensor, sb: torch.Tensor) -> torch.Tensor:
    """block-scaled e4m3 a[M,K] (sa[M,K/128]) @ b[N,K]^T (sb[N/128,K/128]) -> bf16 [M,N]"""
    return F8.gemm_fp8_blockscaled(a, sa, b, sb)


@gemm_fp8.register_fake
def _(a, sa, b, sb):
    return a.new_empty((a.shape[0], b.shape[0]), dtype=torch.bfloat16)


@_op("tdist::ag_gemm_fp8", mutates_args=())
def ag_gemm_fp8(a: torch.Tensor, sa: torch.Tensor, b: torch.Tensor, sb: torch.Tensor, ctx: int) -> torch.Tensor:
    """allgather of block-scaled e4m3 rows and scales fused with the GEMM -> bf16 [M, N/ws]"""
    return F8.ag_gemm_fp8(a, sa, b, sb, _CONTEXTS[ctx])


@ag_gemm_fp8.register_fake
def _(a, sa, b, sb, ctx):
    return a.new_empty((a.shape[0] * _CONTEXTS[ctx].world, b.shape[0]), dtype=torch.bfloat16)


# ---------------------------------------------------------------------------- collectives
@_op("tdist::reduce_scatter", mutates_args=())
def reduce_scatter(x: torch.Tensor, ctx: int) -> torch.Tensor:
    """sum over ranks of x[M,N], rows scattered -> [M/ws, N]"""
    return CO.reduce_scatter_2d_op(x, _CONTEXTS[ctx])


@reduce_scatter.register_fake
def _(x, ctx):
    return x.new_empty((x.shape[0] // _CONTEXTS[ctx].world, x.shape[1]))


@_op("tdist::barrier_all", mutates_args=())
def barrier_all() -> None:
    """device-side barrier of all ranks on the current stream"""
    CO.barrier_all_on_stream()


@barrier_all.register_fake
def _():
    return None


# ---------------------------------------------------------------------------- MoE
@_op("tdist::moe_topk_softmax", mutates_args=())
def moe_topk_softmax(logits: torch.Tensor, topk: int, renormalize: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    ids, w = MU.topk_softmax(logits, topk, renormalize)
    return ids, w


@moe_topk_softmax.register_fake
def _(logits, topk, renormalize):
    return (logits.new_empty((logits.shape[0], topk), dtype=torch.int32),
            logits.new_empty((logits.shape[0], topk), dtype=torch.float32))


@_op("tdist::moe_ag_scatter_align_block_size", mutates_args=())
def moe_ag_scatter_align_block_size(topk_ids: torch.Tensor, num_experts: int, num_ranks: int, num_tokens_per_rank: int,
                                    block_size: int) -> List[torch.Tensor]:
    """(sorted_token_ids, expert_ids, block_barrier_ids, rank_block_num, num_tokens_post_pad); the name the
    reference registers for its CUDA op (csrc/lib/moe_utils.cu)."""
    return list(MU.sort_topk_ids_align_block_size(topk_ids, num_experts, num_ranks, num_tokens_per_rank, block_size))


@moe_ag_scatter_align_block_size.register_fake
def _(topk_ids, num_experts, num_ranks, num_tokens_per_rank, block_size):
    numel = num_tokens_per_rank * topk_ids.shape[1]
    i32 = dict(dtype=torch.int32)
    return [topk_ids.new_empty(((numel + num_experts * (block_size - 1)) * num_ranks,), **i32),
            topk_ids.new_empty(((numel + num_experts) * num_ranks,), **i32),
            topk_ids.new_empty(((numel + num_experts) * num_ranks,), **i32),
            topk_ids.new_empty((num_ranks,), **i32), topk_ids.new_empty((1,), **i32)]


@_op("tdist::moe_dispatch", mutates_args=())
def moe_dispatch(x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, ctx: int
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """fp8 rows, per-128 scales and per-expert counts received by this rank (views of the receive
    buffers are cloned so that the op owns its outputs)"""
    rx, rs, splits = A.moe_dispatch(_CONTEXTS[ctx], x, topk_ids, topk_weights)
    return rx.clone(), rs.clone(), splits.clone()


@moe_dispatch.register_fake
def _(x, topk_ids, topk_weights, ctx):
    c = _CONTEXTS[ctx].ep
    return (x.new_empty((c.rows, c.hidden), dtype=torch.float8_e4m3fn), x.new_empty((c.rows, c.hidden // 128), dtype=torch.float32),
            x.new_empty((c.world, c.experts_per_rank), dtype=torch.int32))


@_op("tdist::moe_combine", mutates_args=())
def moe_combine(expert_out: torch.Tensor, recv_splits: torch.Tensor, ctx: int) -> torch.Tensor:
    return A.moe_combine(_CONTEXTS[ctx], expert_out, recv_splits)


@moe_combine.register_fake
def _(expert_out, recv_splits, ctx):
    c = _CONTEXTS[ctx]
    return expert_out.new_empty((c.ntok, c.hidden))


@_op("tdist::ep_dispatch", mutates_args=())
def ep_dispatch(x: torch.Tensor, topk_ids: torch.Tensor, ctx: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Expert-parallel dispatch into the expert-major layout: ``(rows [capacity, hidden] bf16, recv_splits
    [world, experts_per_rank] int32, num_recv [1] int32)``, cloned so that the op owns its outputs."""
    from .ops import moe_ep as EP
    rows, _, splits, num = EP.ep_dispatch(_CONTEXTS[ctx], x, topk_ids, None)
    return rows.clone(), splits.clone(), num.clone()


@ep_dispatch.register_fake
def _(x, topk_ids, ctx):
    c = _CONTEXTS[ctx]
    return (x.new_empty((c.rows, c.hidden)), x.new_empty((c.world, c.experts_per_rank), dtype=torch.int32),
            x.new_empty((1,), dtype=torch.int32))


@_op("tdist::ep_combine", mutates_args=())
def ep_combine(expert_out: torch.Tensor, ctx: int) -> torch.Tensor:
    """Plain sum of each token's ``topk`` processed rows, read from their owners."""
    from .ops import moe_ep as EP
    return EP.ep_combine(_CONTEXTS[ctx], expert_out, weighted=False)


@ep_combine.register_fake
def _(expert_out, ctx):
    c = _CONTEXTS[ctx]
    return expert_out.new_empty((c.ntok, c.hidden))


# ---------------------------------------------------------------------------- decode attention
@_op("tdist::gqa_fwd_batch_decode", mutates_args=())
def gqa_fwd_batch_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_lens: torch.Tensor,
                         block_table: torch.Tensor, scale: float, soft_cap: float) -> torch.Tensor:
    return FD.gqa_fwd_batch_decode(q, k_cache, v_cache, None, None, kv_lens, block_table, scale, soft_cap)


@gqa_fwd_batch_decode.register_fake
def _(q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap):
    return torch.empty_like(q)


@_op("tdist::gqa_fwd_batch_decode_intra_rank", mutates_args=())
def gqa_fwd_batch_decode_intra_rank(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_lens: torch.Tensor,
                                    block_table: torch.Tensor, scale: float, soft_cap: float) -> torch.Tensor:
    return FD.gqa_fwd_batch_decode_intra_rank(q, k_cache, v_cache, None, None, kv_lens, block_table, scale, soft_cap)


@gqa_fwd_batch_decode_intra_rank.register_fake
def _(q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap):
    return q.new_empty((q.shape[0], q.shape[1], q.shape[2] + 1), dtype=torch.float32)


@_op("tdist::sp_gqa_fwd_batch_decode", mutates_args=())
def sp_gqa_fwd_batch_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, global_kv_lens: torch.Tensor,
                            block_table: torch.Tensor, scale: float, soft_cap: float, ctx: int) -> torch.Tensor:
    return FD.sp_gqa_fwd_batch_decode(_CONTEXTS[ctx], q, k_cache, v_cache, global_kv_lens, block_table, scale, soft_cap)


@sp_gqa_fwd_batch_decode.register_fake
def _(q, k_cache, v_cache, global_kv_lens, block_table, scale, soft_cap, ctx):
    return torch.empty_like(q)


@_op("tdist::lse_combine", mutates_args=())
def lse_combine(partials: torch.Tensor) -> torch.Tensor:
    """[R,B,Hq,D+1] (O || LSE) -> bf16 [B,Hq,D]"""
    return FD.inter_rank_combine(partials, torch.bfloat16)


@lse_combine.register_fake
def _(partials):
    return partials.new_empty(tuple(partials.shape[1:-1]) + (partials.shape[-1] - 1,), dtype=torch.bfloat16)


OP_NAMES = ["gemm", "ag_gemm", "gemm_rs", "gemm_fp8", "ag_gemm_fp8", "group_gemm", "reduce_scatter", "barrier_all", "moe_topk_softmax",
            "moe_ag_scatter_align_block_size", "moe_dispatch", "moe_combine", "ep_dispatch", "ep_combine", "gqa_fwd_batch_decode",
            "gqa_fwd_batch_decode_intra_rank", "sp_gqa_fwd_batch_decode", "lse_combine"]
