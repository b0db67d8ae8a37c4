"""``AllGatherLayer``, ``EPAll2AllLayer`` and ``SpGQAFlashDecodeAttention`` with the reference's
constructor arguments and methods (reference layers/nvidia/low_latency_allgather_layer.py:31-195,
ep_a2a_layer.py:40-240, sp_flash_decode_layer.py:43-184), built on this package's kernels."""
from __future__ import annotations


import torch

from ..ops import collectives as CO
from ..ops import flash_decode as FD
from ..ops import moe_ep as EP
from ..runtime import symm_heap


class AllGatherLayer:
    """Low-latency all-gather with ``stages`` rotating symmetric buffers, so that a call never
    overwrites a buffer a slower rank may still be reading. Every ``forward_*`` takes this rank's
    segment and returns the gathered tensor ``[world, *segment.shape]`` (a view of the stage buffer)."""

    def __init__(self, nnodes: int, world_size: int, rank: int, max_buffer_size: int = 2 * 32 * 1024 * 1024, stages: int = 2,
                 heap=None, group=None, device=None):
        self.nnodes, self.world_size, self.rank, self.stages = nnodes, world_size, rank, max(2, stages)
        self.max_buffer_size = max_buffer_size
        self.group = group
        dev = torch.device(device) if device is not None else (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.device = dev
        heap = heap or symm_heap(group)
        self.buffers = [heap.empty((max_buffer_size,), torch.uint8) for _ in range(self.stages)]
        self.ctxs = [CO.create_fast_allgather_context(rank, 0, world_size, nnodes, max_buffer_size=max_buffer_size, heap=heap,
                                                      group=group, device=dev) for _ in range(self.stages)]
        self.stage = 0

    def _forward(self, segment: torch.Tensor, mode: str, phase: int = 3) -> torch.Tensor:
        nbytes = segment.numel() * segment.element_size()
        total = nbytes * self.world_size
        if total > self.max_buffer_size:
            raise ValueError(f"{total} bytes exceed max_buffer_size {self.max_buffer_size}")
        if phase != 2:
            self.stage = (self.stage + 1) % self.stages
        buf = self.buffers[self.stage].view_as((total,), torch.uint8)
        if phase != 2:
            buf.local[self.rank * nbytes:(self.rank + 1) * nbytes].copy_(segment.contiguous().reshape(-1).view(torch.uint8))
        CO.fast_allgather(buf, self.ctxs[self.stage], mode=mode, phase=phase)
        return buf.local.view(segment.dtype).view(self.world_size, *segment.shape)

    def forward_pull(self, x, **kw): return self._forward(x, "pull", **kw)
    def forward_push_2d(self, x, **kw): return self._forward(x, "push2d", **kw)
    def forward_push_3d(self, x, **kw): return self._forward(x, "push3d", **kw)
    def forward_push_2d_ll(self, x, **kw): return self._forward(x, "push2d_ll", **kw)
    def forward_push_3d_ll(self, x, **kw): return self._forward(x, "push3d_ll", **kw)
    def forward_push_2d_ll_multimem(self, x, **kw): return self._forward(x, "push2d_ll_multimem", **kw)
    def forward_push_numa_2d(self, x, **kw): return self._forward(x, "push_numa_2d", **kw)
    def forward_push_numa_2d_ll(self, x, **kw): return self._forward(x, "push_numa_2d_ll", **kw)
    def forward_push_numa_2d_ll_multinode(self, x, **kw): return self._forward(x, "push_numa_2d_ll_multinode", **kw)


class EPAll2AllLayer:
    """Expert-parallel token exchange (reference layers/nvidia/ep_a2a_layer.py:40-240).

    ``dispatch(input[T,hidden], exp_indices[T,topk])`` returns the rows this rank's experts have to process, grouped
    by local expert and, inside an expert, by source rank (each group in the source's token order);
    ``combine(x)`` reads the processed rows back from their owners and sums each token's ``topk`` copies. Both are
    one kernel launch (``csrc/kernels/moe_ep.cu``) and neither synchronises with the host: the receive buffer is
    returned at its full capacity, ``num_recv`` (device int32 ``[1]``) says how many leading rows are live,
    ``recv_splits`` ``[world, experts_per_rank]`` and ``recv_offset`` ``[experts_per_rank, world]`` describe the
    groups. ``dispatch(..., exact=True)`` reads the count back and returns exactly ``[num_recv, hidden]`` like the
    reference (one host synchronisation)."""

    def __init__(self, ep_group, max_tokens: int, hidden: int, topk: int, rank: int, num_tot_experts: int,
                 local_world_size: int, world_size: int, dtype=torch.bfloat16, num_sm: int = 20, heap=None, device=None,
                 capacity=None, align: int = 1):
        if dtype != torch.bfloat16:
            raise ValueError("the expert-parallel exchange moves bf16 rows")
        self.group, self.rank, self.world_size = ep_group, rank, world_size
        self.hidden, self.topk, self.num_experts = hidden, topk, num_tot_experts
        self.epr = num_tot_experts // world_size
        self.ctx = EP.create_ep_context(max_tokens, hidden, topk, num_tot_experts, rank, world_size, quant=False, compact=True,
                                        align=align, capacity=capacity, heap=heap, group=ep_group, device=device)

    @property
    def num_recv(self) -> torch.Tensor:
        return self.ctx.num_recv

    @property
    def recv_splits(self) -> torch.Tensor:
        return self.ctx.recv_splits

    @property
    def recv_offset(self) -> torch.Tensor:
        return self.ctx.recv_offset

    def dispatch(self, input: torch.Tensor, exp_indices: torch.Tensor, phase: int = 7, exact: bool = False):
        """``phase`` bits (emulated ranks run them one after the other): 1 publish counts, 2 send, 4 wait."""
        recv, _, _, num_recv = EP.ep_dispatch(self.ctx, input, exp_indices, None, phase=phase)
        if not (phase & 4):
            return None
        return recv[: int(num_recv)] if exact else recv

    def output_buffer(self) -> torch.Tensor:
        """Symmetric buffer ``[capacity, hidden]`` for the processed rows of the call in flight: write row ``i`` of the
        experts' output where row ``i`` of the dispatched rows was, then call ``combine()`` without an argument."""
        return EP.expert_out_buffer(self.ctx)

    def combine(self, x=None, phase: int = 3) -> torch.Tensor:
        """Sum of each token's ``topk`` processed copies, ``[T, hidden]``. ``x`` is ``output_buffer()`` (or nothing), or
        any ``[rows, hidden]`` bf16 tensor in the dispatched row order, which is first copied there."""
        return EP.ep_combine(self.ctx, x, weighted=False, phase=phase)


class SpGQAFlashDecodeAttention:
    """Sequence-parallel GQA decode attention: every rank owns a contiguous shard of each sequence's
    KV in its own paged cache; ``forward`` returns attention over the whole sequence on every rank."""

    def __init__(self, rank: int, node: int, num_ranks: int, num_nodes: int, num_q_heads: int, num_kv_heads: int, q_head_dim: int,
                 v_head_dim: int, page_size: int = 1, scale: float = 1.0, soft_cap: float = 0.0, max_allowed_batch: int = 1,
                 thrink_buffer_threshold: int = 500, stages: int = 20, heap=None, group=None, device=None,
                 cuda_graph_safe: bool = False):
        """``cuda_graph_safe`` keeps the call number on the device so that ``forward`` can be captured and replayed."""
        if q_head_dim != v_head_dim:
            raise ValueError("q and v head dims must match")
        self.rank, self.num_ranks = rank, num_ranks
        self.scale, self.soft_cap = scale, soft_cap
        self.ctx = FD.create_sp_decode_context(rank, num_ranks, max_allowed_batch, num_q_heads, q_head_dim, heap=heap,
                                               group=group, device=device, device_epoch=cuda_graph_safe)

    def forward(self, q, k_cache, v_cache, global_kv_lens, block_table, phase: int = 3):
        return FD.sp_gqa_fwd_batch_decode(self.ctx, q, k_cache, v_cache, global_kv_lens, block_table, self.scale,
                                          self.soft_cap, phase=phase)

    __call__ = forward
