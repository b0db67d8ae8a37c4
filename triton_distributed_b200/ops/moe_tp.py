"""Tensor-parallel MoE ops: grouped GEMM on tcgen05, AllGather + GroupGEMM, GroupGEMM + top-k
reduce + ReduceScatter.

Public surface (names of the reference):

* ``select_experts(pg, num_ranks, topk, input_dtype, device, router_logits)``
  (reference kernels/nvidia/moe_reduce_rs.py:180-197)
* ``create_ag_group_gemm_intra_node_context`` / ``ag_group_gemm_intra_node(a[M/ws,K], b[E,K,N/ws], ctx)
  -> [M*topk, N/ws]`` (reference kernels/nvidia/allgather_group_gemm.py:555-691)
* ``create_moe_rs_context`` / ``moe_reduce_rs(rank, world, local_world, a[M*topk,K/ws], b[E,K/ws,N], ctx)
  -> [M/ws, N]`` (reference kernels/nvidia/moe_reduce_rs.py:280-361,889-1029)
* ``group_gemm(a_sorted, b[E,N,K], expert_ids, num_blocks)`` — the grouped tcgen05 GEMM itself.

Pipeline on CUDA (each stage one hand-written kernel): all-gather of the token shards (push kernel
over NVLink) -> block-aligned expert sort (``moe_align_block_size``) -> row gather into the sorted,
128-row-padded layout -> grouped GEMM (the persistent tcgen05 kernel picking B[expert] per 128-row
block) -> top-k weighted reduce fused into the reduce-scatter kernel (each token's expert outputs are reduced
straight into the owning rank's staging). The all-gather and the grouped GEMM are separate launches.

CPU tensors run a torch restatement (masked per-expert matmul, the reference's own oracle:
test/nvidia/test_ag_moe.py:24-39).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import _lib
from ..runtime import counters_clean, symm_heap
from . import collectives as CO
from . import gemm as G
from . import moe_utils as MU

GROUP_BLOCK_M = 128
# How AllGather + GroupGEMM (and the A side of GroupGEMM + reduce-scatter) run:
#   "staged"   all-gather kernel, row-gather kernel, TMA-fed grouped GEMM, un-sort kernel (four launches, no overlap);
#   "fused"    (default) the all-gather only sends; ONE grouped-GEMM launch whose first CTAs copy the rows of each
#              128-row block into the sorted staging matrix as the source rank's segment arrives (a flag per block),
#              whose other CTAs feed on that matrix with TMA block by block, starting at this rank's own tokens, and
#              whose epilogue stores every row straight to its (token, k) position: gather, all-gather wait and
#              un-sort overlap the MMAs;
#   "cp_async" the grouped GEMM's producer warps gather the rows themselves with 16-byte cp.async copies (kept for
#              comparison: 2.2x slower than "staged", the L2 request rate saturates long before TMA does).
AG_GROUP_GEMM_MODE = "fused"
# All-gather feeding the one-launch forms. "push" sends to all peers at once: every segment lands at the end of the
# all-gather. "push_ordered" sends the segments in the order the grouped GEMM of each peer reaches them (rank + 1's
# first), one fence per destination more. "auto": ordered above four ranks. Measured at tp4 (8192 tokens, hidden 4096,
# 3584 columns per rank), where the GEMM of a rank's own blocks (~110 us) outlasts the whole all-gather (~100 us): 602 us
# ordered, 585 us at once. At tp8 the own blocks take ~35 us of a ~145 us all-gather, which is what the ordered form is
# for; that case has not been timed.
AG_PUSH_MODE = os.environ.get("TDIST_MOE_AG_PUSH_MODE", "auto")


def _ag_push_mode(world: int) -> str:
    if AG_PUSH_MODE != "auto":
        return AG_PUSH_MODE
    return "push_ordered" if world > 4 else "push"
FUSED_AG_GROUP_GEMM = False   # legacy switch: True selects "cp_async"
FUSED_TOPK_RS = True   # False: separate top-k reduce kernel, then the plain reduce-scatter (for A/B checks)
launch_count = 0


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def select_experts(pg, num_ranks: int, topk: int, input_dtype, device, router_logits: torch.Tensor
                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax -> top-k on this rank's tokens, then all-gather ids and weights of every rank's
    tokens (NCCL / gloo: this is set-up, not a hot path). Returns ``(full_topk_ids int32 [M, topk],
    full_topk_weight [M, topk])``."""
    ids, w = MU.topk_softmax(router_logits, topk)
    if num_ranks > 1:
        full_ids = torch.empty((ids.shape[0] * num_ranks, topk), dtype=ids.dtype, device=ids.device)
        full_w = torch.empty((w.shape[0] * num_ranks, topk), dtype=w.dtype, device=w.device)
        dist.all_gather_into_tensor(full_ids, ids, group=pg)
        dist.all_gather_into_tensor(full_w, w, group=pg)
        return full_ids, full_w.to(input_dtype)
    return ids, w.to(input_dtype)


# ---------------------------------------------------------------------------- grouped GEMM
def gather_rows(src: torch.Tensor, index: torch.Tensor, div: int, limit: int, want_inverse: bool = False):
    """``dst[p] = src[index[p] // div]`` (zeros where ``index[p]`` is padding); optionally also the
    inverse map ``pos_of[index[p]] = p``."""
    global launch_count
    rows_out = index.shape[0]
    dst = torch.empty((rows_out, src.shape[1]), dtype=src.dtype, device=src.device)
    pos_of = torch.zeros(limit, dtype=torch.int32, device=src.device) if want_inverse else None
    if src.device.type != "cuda":
        live = (index >= 0) & (index < limit)
        rows = torch.where(live, index.long() // div, torch.zeros_like(index).long())
        dst.copy_(src[rows] * live.unsqueeze(-1).to(src.dtype))
        if want_inverse:
            pos_of[index[live].long()] = torch.arange(rows_out, dtype=torch.int32)[live]
        return dst, pos_of
    _lib.check(_lib.lib().tdist_gather_rows(src.data_ptr(), index.data_ptr(), rows_out, div, limit,
                                            src.shape[1] * src.element_size(), dst.data_ptr(),
                                            pos_of.data_ptr() if want_inverse else None, _stream(src)), "tdist_gather_rows")
    launch_count += 1
    return dst, pos_of


def topk_reduce(y: torch.Tensor, pos_of: torch.Tensor, weights: Optional[torch.Tensor], ntok: int, topk: int) -> torch.Tensor:
    """``out[t] = sum_k weights[t,k] * y[pos_of[t*topk+k]]`` (fp32 accumulation)."""
    global launch_count
    out = torch.empty((ntok, y.shape[1]), dtype=y.dtype, device=y.device)
    if y.device.type != "cuda" or y.dtype != torch.bfloat16:
        rows = y[pos_of.long()].float().view(ntok, topk, -1)
        w = weights.float().view(ntok, topk, 1) if weights is not None else 1.0
        return (rows * w).sum(1).to(y.dtype)
    w = weights.float().contiguous() if weights is not None else None
    _lib.check(_lib.lib().tdist_topk_reduce(y.data_ptr(), pos_of.data_ptr(), w.data_ptr() if w is not None else None,
                                            ntok, topk, y.shape[1] * 2, out.data_ptr(), _stream(y)), "tdist_topk_reduce")
    launch_count += 1
    return out


def group_gemm(a_sorted: torch.Tensor, b: torch.Tensor, expert_ids: torch.Tensor, num_blocks: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[i*128:(i+1)*128] = a_sorted[i*128:(i+1)*128] @ b[expert_ids[i]].T`` for every live
    128-row block. ``a_sorted`` ``[blocks*128, K]``, ``b`` ``[E, N, K]`` (K contiguous), ``num_blocks``
    an int32 device scalar (blocks past it are padding and are skipped)."""
    rows, K = a_sorted.shape
    E, N, _ = b.shape
    if rows % GROUP_BLOCK_M:
        raise ValueError("grouped GEMM rows must be a multiple of 128")
    if a_sorted.device.type != "cuda":
        o = torch.zeros((rows, N), dtype=a_sorted.dtype)
        nb = rows // GROUP_BLOCK_M if num_blocks is None else int(num_blocks)
        for i in range(nb):
            blk = slice(i * GROUP_BLOCK_M, (i + 1) * GROUP_BLOCK_M)
            o[blk] = (a_sorted[blk].float() @ b[int(expert_ids[i])].float().t()).to(o.dtype)
        return o
    G._check_operands(a_sorted, b.view(E * N, K))
    c = out if out is not None else torch.empty((rows, N), dtype=a_sorted.dtype, device=a_sorted.device)
    g = G._base_args(a_sorted, b.view(E * N, K), 1, 0, _lib.GEMM_PLAIN)
    g.n = N
    g.c = c.data_ptr()
    g.m_per_rank = rows
    g.epoch = 1
    g.expert_ids = expert_ids.data_ptr()
    g.num_m_blocks = num_blocks.data_ptr() if num_blocks is not None else None
    g.num_experts = E
    G._launch(g)
    return c


def staging_flags(rows: int, device) -> torch.Tensor:
    """Flag words of a staged row gather over up to ``rows`` sorted rows: one int32 per 128-row block (the call number at
    which its rows were staged) followed by the kernel's own counters (4 + one per block). Zero before the first call."""
    blocks = (rows + GROUP_BLOCK_M - 1) // GROUP_BLOCK_M
    return torch.zeros(2 * blocks + 4, dtype=torch.int32, device=device)


def group_gemm_gather(a: torch.Tensor, row_index: torch.Tensor, b: torch.Tensor, expert_ids: torch.Tensor,
                      num_blocks: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                      block_src: Optional[torch.Tensor] = None, src_flags: Optional[torch.Tensor] = None, src_epoch: int = 0,
                      src_rank: int = 0, src_world: int = 1, staging: Optional[torch.Tensor] = None,
                      block_ready: Optional[torch.Tensor] = None, epoch: int = 1, block_rot: Optional[torch.Tensor] = None,
                      c_scatter: Optional[torch.Tensor] = None, c_rows: int = 0) -> torch.Tensor:
    """Grouped GEMM whose A rows are gathered inside the kernel: ``out[r] = a[row_index[r]] @ b[expert_ids[r // 128]].T``
    (rows with ``row_index >= a.shape[0]`` are padding). With ``block_src`` the rows of 128-row
    block ``i`` come from rank ``block_src[i]``'s segment of an all-gather that may still be in flight: the kernel
    waits for that rank's arrival flag (``src_flags[rank] >= src_epoch``) before loading them, so blocks of ranks
    that have arrived compute while later segments are still on the wire.

    With ``staging`` (``[rows, K]`` workspace) and ``block_ready`` (from :func:`staging_flags`; ``epoch`` strictly increasing
    per call) the launch copies the rows into ``staging`` itself (all threads for the first wave of tiles, then the
    epilogue warps while they wait for accumulators) and the GEMM is fed by TMA; without them the producer warps copy
    the rows with cp.async.
    ``block_rot`` (device int32 scalar): block the schedule starts at. ``c_scatter`` (int32 per sorted row): the
    epilogue stores row ``r`` of the product at row ``c_scatter[r]`` of ``out`` (``[c_rows, N]``), dropping rows whose
    index is not below ``c_rows``."""
    rows = row_index.shape[0]
    E, N, K = b.shape
    if rows % GROUP_BLOCK_M:
        raise ValueError("grouped GEMM rows must be a multiple of 128")
    if a.device.type != "cuda":
        padded = torch.cat([a, a.new_zeros((1, K))])
        prod = group_gemm(padded[row_index.long().clamp(max=a.shape[0])], b, expert_ids, num_blocks)
        if c_scatter is None:
            return prod
        o = out if out is not None else torch.zeros((c_rows, N), dtype=a.dtype)
        live = c_scatter.long() < c_rows
        o[c_scatter.long()[live]] = prod[live]
        return o
    G._check_operands(a, b.view(E * N, K))
    if c_scatter is not None:
        c = out if out is not None else torch.empty((c_rows, N), dtype=a.dtype, device=a.device)
    else:
        c = out if out is not None else torch.empty((rows, N), dtype=a.dtype, device=a.device)
    g = G._base_args(a, b.view(E * N, K), 1, 0, _lib.GEMM_PLAIN)
    g.n = N
    g.c = c.data_ptr()
    g.m_per_rank = rows
    g.epoch = epoch
    g.expert_ids = expert_ids.data_ptr()
    g.num_m_blocks = num_blocks.data_ptr() if num_blocks is not None else None
    g.num_experts = E
    g.cta_pair = 0
    g.a_gather = row_index.data_ptr()
    g.a_gather_rows = a.shape[0]
    if staging is not None:
        if block_ready is None or staging.shape[0] < rows or staging.shape[1] != K or staging.dtype != a.dtype:
            raise ValueError("staging must be [rows, K] of a's dtype, with block_ready")
        blocks = rows // GROUP_BLOCK_M
        if block_ready.numel() < 2 * blocks + 4 or block_ready.dtype != torch.int32:
            raise ValueError("block_ready must come from staging_flags(rows)")
        # flags first; the kernel's counters (4 + one per block) after the flags of the blocks the buffer was sized for
        g.gather_dst, g.block_ready = staging.data_ptr(), block_ready.data_ptr()
        g.gather_counter = block_ready.data_ptr() + 4 * ((block_ready.numel() - 4) // 2)
        counters_clean(block_ready, (block_ready.numel() - 4) // 2)
    if block_rot is not None:
        g.block_rot = block_rot.data_ptr()
    if c_scatter is not None:
        g.c_scatter, g.c_rows = c_scatter.data_ptr(), c_rows
    if block_src is not None:
        g.block_src = block_src.data_ptr()
        g.src_flags = src_flags.data_ptr()
        g.src_epoch = src_epoch
        g.src_rank, g.src_world = src_rank, src_world
    G._launch(g)
    return c


# ---------------------------------------------------------------------------- AG + GroupGEMM
@dataclass
class MoEAllGatherGroupGEMMTensorParallelContext:
    rank: int
    world: int
    num_experts: int
    topk: int
    max_M: int
    K: int
    full_topk_ids: torch.Tensor
    group: object = None
    gather_buf: Optional[object] = None          # symmetric [max_M, K]
    ag_ctx: Optional[CO.FastAllGatherContext] = None
    sorted_ids: Optional[torch.Tensor] = None
    expert_ids: Optional[torch.Tensor] = None
    block_barrier_ids: Optional[torch.Tensor] = None
    rank_block_num: Optional[torch.Tensor] = None
    num_blocks: Optional[torch.Tensor] = None    # int32 [1]: live 128-row blocks
    b_nk: Optional[torch.Tensor] = None          # [E, N, K] copy of the weights (K contiguous)
    row_index: Optional[torch.Tensor] = None     # int32 [sorted rows]: token of every sorted row (padding = M)
    pos_of: Optional[torch.Tensor] = None        # int32 [M * topk]: sorted row of every (token, k) pair
    staging: Optional[torch.Tensor] = None       # [sorted rows, K]: the rows in sorted order, filled inside the GEMM launch
    block_ready: Optional[torch.Tensor] = None   # int32 per 128-row block: call number at which its rows were staged
    block_rot: Optional[torch.Tensor] = None     # int32 [1]: first block of this rank's own tokens
    gemm_calls: int = 0
    calls: int = 0


def sort_topk_ids_align_block_size(topk_ids, num_experts, num_ranks, num_tokens_per_rank, block_size, moe_stream=None):
    return MU.sort_topk_ids_align_block_size(topk_ids, num_experts, num_ranks, num_tokens_per_rank, block_size, moe_stream)


def create_ag_group_gemm_intra_node_context(tp_pg, A: torch.Tensor, B: torch.Tensor, full_topk_ids: torch.Tensor,
                                            num_experts: int, max_M: int = 2 ** 14, BLOCK_M: int = 128, BLOCK_N: int = 256,
                                            BLOCK_K: int = 64, GROUP_SIZE_M: int = 8, stages: int = 4, warps: int = 8,
                                            ag_stream=None, group_gemm_stream=None, rank: Optional[int] = None,
                                            num_ranks: Optional[int] = None, heap=None
                                            ) -> MoEAllGatherGroupGEMMTensorParallelContext:
    """``A`` is this rank's ``[M/ws, K]`` token shard, ``B`` ``[E, K, N/ws]`` the expert weights,
    ``full_topk_ids`` ``[M, topk]`` the routing of ALL ranks' tokens."""
    rank = dist.get_rank(tp_pg) if rank is None else rank
    world = dist.get_world_size(tp_pg) if num_ranks is None else num_ranks
    M, topk = full_topk_ids.shape
    K = A.shape[1]
    ctx = MoEAllGatherGroupGEMMTensorParallelContext(rank, world, num_experts, topk, max(max_M, M), K,
                                                     full_topk_ids.to(torch.int32).contiguous(), group=tp_pg)
    tpr = M // world
    (sorted_ids, ctx.expert_ids, ctx.block_barrier_ids, ctx.rank_block_num, post_pad) = \
        MU.sort_topk_ids_align_block_size(ctx.full_topk_ids, num_experts, world, tpr, GROUP_BLOCK_M)
    # set-up time: read the padded length once so that the per-call gather and GEMM cover only live blocks
    ctx.sorted_ids = sorted_ids[: int(post_pad)].contiguous()
    ctx.num_blocks = (post_pad // GROUP_BLOCK_M).to(torch.int32)
    ctx.b_nk = B.transpose(1, 2).contiguous()
    # static routing: the gather index of the fused kernel and the inverse permutation of its output
    numel = M * topk
    ctx.row_index = torch.div(ctx.sorted_ids, topk, rounding_mode="floor").to(torch.int32).contiguous()   # padding numel -> M
    valid = ctx.sorted_ids < numel
    ctx.pos_of = torch.zeros(numel, dtype=torch.int32, device=ctx.sorted_ids.device)
    ctx.pos_of[ctx.sorted_ids[valid].long()] = torch.arange(ctx.sorted_ids.numel(), dtype=torch.int32, device=ctx.sorted_ids.device)[valid]
    if A.device.type == "cuda":
        ctx.staging = torch.empty((ctx.sorted_ids.numel(), K), dtype=A.dtype, device=A.device)
        ctx.block_ready = staging_flags(ctx.sorted_ids.numel(), A.device)
        before = torch.cumsum(ctx.rank_block_num, 0) - ctx.rank_block_num
        ctx.block_rot = before[rank:rank + 1].to(torch.int32).contiguous()
    if A.device.type == "cuda" and world > 1:
        heap = heap or symm_heap(tp_pg)
        # two gather buffers, alternated per call: a rank that is one call ahead pushes into the other one
        ctx.gather_buf = heap.empty((2, ctx.max_M, K), A.dtype)
        ctx.ag_ctx = CO.create_fast_allgather_context(rank, 0, world, 1, max_buffer_size=ctx.max_M * K * A.element_size(),
                                                      heap=heap, group=tp_pg, device=A.device)
    return ctx


def ag_group_gemm_intra_node(a: torch.Tensor, b: torch.Tensor, ctx: MoEAllGatherGroupGEMMTensorParallelContext,
                             phase: int = 3) -> torch.Tensor:
    """``C[M*topk, N/ws]``: row ``t*topk+k`` = ``allgather(a)[t] @ b[full_topk_ids[t,k]]``."""
    mpr, K = a.shape
    M = mpr * ctx.world
    numel = M * ctx.topk
    if a.device.type != "cuda":
        full = a
        if ctx.world > 1:
            full = torch.empty((M, K), dtype=a.dtype)
            dist.all_gather_into_tensor(full, a.contiguous(), group=ctx.group)
        out = torch.empty((numel, b.shape[2]), dtype=a.dtype)
        ids = ctx.full_topk_ids.reshape(-1).long()
        rows = full[torch.arange(numel) // ctx.topk].float()
        for e in range(ctx.num_experts):
            m = ids == e
            out[m] = (rows[m] @ b[e].float()).to(a.dtype)
        return out
    b_nk = ctx.b_nk if ctx.b_nk is not None else b.transpose(1, 2).contiguous()
    if ctx.world > 1:
        if phase != 2:
            ctx.calls += 1
        half = ctx.calls & 1
        nbytes = M * K * a.element_size()
        buf = ctx.gather_buf.view_as((M, K), a.dtype, offset_bytes=half * ctx.max_M * K * a.element_size())
        if phase != 2:
            buf.local[ctx.rank * mpr:(ctx.rank + 1) * mpr].copy_(a)
        mode = "cp_async" if FUSED_AG_GROUP_GEMM else AG_GROUP_GEMM_MODE
        if mode != "staged":
            # send half of the all-gather only; the grouped GEMM launch gathers its A rows itself and waits, block by
            # block, for the arrival flag of the rank the block's tokens come from
            if phase != 2:
                CO.fast_allgather(buf, ctx.ag_ctx, mode=_ag_push_mode(ctx.world), phase=1)
            if phase == 1:
                return None
            src = dict(block_src=ctx.block_barrier_ids, src_flags=ctx.ag_ctx.signal.local, src_epoch=ctx.ag_ctx.epoch,
                       src_rank=ctx.rank, src_world=ctx.world)
            if mode == "fused":
                return _fused_group_gemm(ctx, buf.local, b_nk, numel, **src)
            c_sorted = group_gemm_gather(buf.local, ctx.row_index, b_nk, ctx.expert_ids, ctx.num_blocks, **src)
            out, _ = gather_rows(c_sorted, ctx.pos_of, 1, c_sorted.shape[0])
            return out
        CO.fast_allgather(buf, ctx.ag_ctx, mode="push", phase=phase)
        if phase == 1:
            return None
        full = buf.local
    else:
        full = a
    mode = "cp_async" if FUSED_AG_GROUP_GEMM else AG_GROUP_GEMM_MODE
    if mode == "fused":
        return _fused_group_gemm(ctx, full, b_nk, numel)
    if mode == "cp_async":
        c_sorted = group_gemm_gather(full, ctx.row_index, b_nk, ctx.expert_ids, ctx.num_blocks)
        out, _ = gather_rows(c_sorted, ctx.pos_of, 1, c_sorted.shape[0])
        return out
    a_sorted, pos_of = gather_rows(full, ctx.sorted_ids, ctx.topk, numel, want_inverse=True)
    c_sorted = group_gemm(a_sorted, b_nk, ctx.expert_ids, ctx.num_blocks)
    out, _ = gather_rows(c_sorted, pos_of, 1, c_sorted.shape[0])
    return out


def _fused_group_gemm(ctx: MoEAllGatherGroupGEMMTensorParallelContext, full: torch.Tensor, b_nk: torch.Tensor, numel: int, **src):
    """One launch: the kernel stages the rows block by block itself (all threads for the first wave, then the epilogue
    warps between accumulators), TMA-fed MMAs start at this rank's own blocks, the epilogue stores every row at its
    (token, k) position."""
    ctx.gemm_calls += 1
    return group_gemm_gather(full, ctx.row_index, b_nk, ctx.expert_ids, ctx.num_blocks, staging=ctx.staging,
                             block_ready=ctx.block_ready, epoch=ctx.gemm_calls, block_rot=ctx.block_rot,
                             c_scatter=ctx.sorted_ids, c_rows=numel, **src)


# ---------------------------------------------------------------------------- GroupGEMM + reduce + RS
@dataclass
class MoEReduceRSContext:
    rank: int
    world: int
    max_token_num: int
    hidden_dim: int
    num_experts: int
    topk: int
    full_topk_ids: torch.Tensor
    full_topk_weight: torch.Tensor
    group: object = None
    sorted_ids: Optional[torch.Tensor] = None
    expert_ids: Optional[torch.Tensor] = None
    num_blocks: Optional[torch.Tensor] = None
    rs_ctx: Optional[CO.ReduceScatter2DContext] = None
    b_nk: Optional[torch.Tensor] = None   # [E, N, K/ws] copy of the weights, made on first use
    pos_of: Optional[torch.Tensor] = None        # int32 [M * topk]: sorted row of every (token, k) pair
    staging: Optional[torch.Tensor] = None       # [sorted rows, K/ws], allocated on first use
    block_ready: Optional[torch.Tensor] = None
    gemm_calls: int = 0
    _partial: Optional[torch.Tensor] = None


def create_moe_rs_context(pg, local_rank: int, world_size: int, local_world_size: int, max_token_num: int, hidden_dim: int,
                          num_experts: int, topk: int, input_dtype, output_dtype, device, moe_block_size: int = 128,
                          router_logits: Optional[torch.Tensor] = None, full_topk_ids: Optional[torch.Tensor] = None,
                          full_topk_weight: Optional[torch.Tensor] = None, heap=None) -> MoEReduceRSContext:
    """Routing comes either from ``router_logits`` of this rank's tokens (then ``select_experts``
    gathers everybody's) or directly as ``full_topk_ids`` / ``full_topk_weight`` ``[M, topk]``."""
    if full_topk_ids is None:
        full_topk_ids, full_topk_weight = select_experts(pg, world_size, topk, input_dtype, device, router_logits)
    M = full_topk_ids.shape[0]
    ctx = MoEReduceRSContext(local_rank, world_size, max(max_token_num, M), hidden_dim, num_experts, topk,
                             full_topk_ids.to(torch.int32).contiguous(), full_topk_weight.float().contiguous(), group=pg)
    # one "rank" in the aligned sort: the reduction is over all tokens, ordering by source is irrelevant
    sorted_ids, ctx.expert_ids, _bb, _rbn, post_pad = MU.sort_topk_ids_align_block_size(
        ctx.full_topk_ids, num_experts, 1, M, GROUP_BLOCK_M)
    ctx.sorted_ids = sorted_ids[: int(post_pad)].contiguous()
    ctx.num_blocks = (post_pad // GROUP_BLOCK_M).to(torch.int32)
    numel = M * topk
    valid = ctx.sorted_ids < numel
    ctx.pos_of = torch.zeros(numel, dtype=torch.int32, device=ctx.sorted_ids.device)
    ctx.pos_of[ctx.sorted_ids[valid].long()] = torch.arange(ctx.sorted_ids.numel(), dtype=torch.int32, device=ctx.sorted_ids.device)[valid]
    ctx.rs_ctx = CO.create_reduce_scater_2d_ctx(ctx.max_token_num, hidden_dim, local_rank, world_size, dtype=output_dtype,
                                                heap=heap, group=pg, device=device)
    return ctx


def moe_reduce_rs(rank: int, world_size: int, local_world_size: int, a: torch.Tensor, b: torch.Tensor,
                  ctx: MoEReduceRSContext, dump_ir: bool = False, debug_sync: bool = False, do_initial_sync: bool = True,
                  do_final_sync: bool = True, phase: int = 3) -> torch.Tensor:
    """``a`` ``[M*topk, K/ws]`` (row ``t*topk+k`` = token t's input to its k-th expert), ``b``
    ``[E, K/ws, N]``. Returns this rank's ``[M/ws, N]`` rows of
    ``sum_ranks sum_k w[t,k] * a[t*topk+k] @ b[ids[t,k]]``."""
    numel, _ = a.shape
    M = numel // ctx.topk
    N = b.shape[2]
    if a.device.type != "cuda":
        ids = ctx.full_topk_ids.reshape(-1).long()
        y = torch.empty((numel, N), dtype=torch.float32)
        for e in range(ctx.num_experts):
            m = ids == e
            y[m] = a[m].float() @ b[e].float()
        part = (y.view(M, ctx.topk, N) * ctx.full_topk_weight.view(M, ctx.topk, 1)).sum(1).to(a.dtype)
        return CO.reduce_scatter_2d_op(part, ctx.rs_ctx)
    if phase != 2:
        if ctx.b_nk is None:
            ctx.b_nk = b.transpose(1, 2).contiguous()
        if AG_GROUP_GEMM_MODE == "fused":
            # the sort of the rows by expert happens inside the grouped-GEMM launch (in-launch row staging + TMA-fed MMAs)
            if ctx.staging is None or ctx.staging.shape[1] != a.shape[1] or ctx.staging.dtype != a.dtype:
                ctx.staging = torch.empty((ctx.sorted_ids.numel(), a.shape[1]), dtype=a.dtype, device=a.device)
                ctx.block_ready = staging_flags(ctx.sorted_ids.numel(), a.device)
                ctx.gemm_calls = 0
            ctx.gemm_calls += 1
            y = group_gemm_gather(a, ctx.sorted_ids, ctx.b_nk, ctx.expert_ids, ctx.num_blocks, staging=ctx.staging,
                                  block_ready=ctx.block_ready, epoch=ctx.gemm_calls)
            ctx._partial = (y, ctx.pos_of)
        else:
            a_sorted, pos_of = gather_rows(a, ctx.sorted_ids, 1, numel, want_inverse=True)
            ctx._partial = (group_gemm(a_sorted, ctx.b_nk, ctx.expert_ids, ctx.num_blocks), pos_of)
    y_sorted, pos_of = ctx._partial
    if FUSED_TOPK_RS and y_sorted.dtype == torch.bfloat16 and M % world_size == 0:
        # top-k weighted reduce and reduce-scatter in one kernel: the [M, N] partial is never written
        out = CO.topk_reduce_scatter(y_sorted, pos_of, ctx.full_topk_weight, M, ctx.topk, ctx.rs_ctx, phase=phase)
    else:
        out = CO.reduce_scatter_2d_op(topk_reduce(y_sorted, pos_of, ctx.full_topk_weight, M, ctx.topk), ctx.rs_ctx, phase=phase)
    if debug_sync:
        torch.cuda.synchronize()
    return out


# reference names of the multi-node variants (allgather_group_gemm.py:694-823): one NVSwitch node is one level
def create_ag_group_gemm_inter_node_context(tp_pg, A, B, full_topk_ids, num_experts, **kw):
    world = kw.get("num_ranks") or dist.get_world_size(tp_pg)
    if world > 8:
        raise NotImplementedError("multi-node AG + GroupGEMM is not built: one NVSwitch node (up to 8 ranks) is the target")
    return create_ag_group_gemm_intra_node_context(tp_pg, A, B, full_topk_ids, num_experts, **kw)


ag_group_gemm_inter_node = ag_group_gemm_intra_node
