"""``AllGatherLayer``, ``EPAll2AllLayer`` and ``SpGQAFlashDecodeAttention`` with the reference's
constructor arguments and methods (reference layers/nvidia/low_latency_allgather_layer.py:31-195,
ep_a2a_layer.py:40-240, sp_flash_decode_layer.py:43-184), built on this package's kernels."""
from __future__ import annotations


import torch

from ..ops import all_to_all as A
from ..ops import collectives as CO
from ..ops import flash_decode as FD
from ..ops import moe_utils as MU
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
    """Expert-parallel token exchange: ``dispatch(input[T,hidden], exp_indices[T,topk])`` returns the
    rows this rank's experts have to process, grouped by local expert and, inside an expert, by
    source rank; ``combine(x)`` sends the processed rows back and sums each token's ``topk`` copies."""

    def __init__(self, ep_group, max_tokens: int, hidden: int, topk: int, rank: int, num_tot_experts: int,
                 local_world_size: int, world_size: int, dtype=torch.bfloat16, num_sm: int = 20, heap=None, device=None):
        self.group, self.rank, self.world_size = ep_group, rank, world_size
        self.hidden, self.topk, self.num_experts = hidden, topk, num_tot_experts
        self.epr = num_tot_experts // world_size
        self.max_m = max_tokens * topk
        self.dtype = dtype
        self.d_ctx = A.create_all_to_all_context(self.max_m, hidden, rank, num_tot_experts, world_size, self.epr, dtype=dtype,
                                                 heap=heap, group=ep_group, device=device)
        self.c_ctx = A.create_all_to_all_context(self.max_m, hidden, rank, num_tot_experts, world_size, self.epr, dtype=dtype,
                                                 heap=heap, group=ep_group, device=device)
        self._routing = None
        self._ids = None
        self._perm = None
        self._splits = None
        self._ntok = 0

    def dispatch(self, input: torch.Tensor, exp_indices: torch.Tensor, phase: int = 3):
        T = input.shape[0]
        if phase != 2:
            self._ids = exp_indices.to(torch.int32).contiguous()
            self._routing = MU.route(self._ids, self.num_experts)
            self._ntok = T
            self._send = input[self._routing.sorted_token.long()].contiguous()
        splits, recv, _ = A.fast_all_to_all(self.d_ctx, self._send, self._routing.cumsum, None, phase=phase)
        if phase == 1:
            return None
        # receive layout is [source rank][local expert]; regroup to [local expert][source rank]
        W, epr, mm = self.world_size, self.epr, self.max_m
        sp = splits.view(W, epr).long()
        start_in_src = torch.cumsum(sp, 1) - sp                              # [W, epr] offset inside the source's slot
        src_base = (torch.arange(W, device=sp.device) * mm).unsqueeze(1)
        counts = sp.t().reshape(-1)                                          # (expert, src) order
        starts = (src_base + start_in_src).t().reshape(-1)
        total = int(counts.sum())
        seg = torch.repeat_interleave(torch.arange(W * epr, device=sp.device), counts, output_size=total)
        first = torch.cumsum(counts, 0) - counts
        self._perm = starts[seg] + (torch.arange(total, device=sp.device) - first[seg])
        self._splits = splits
        return recv[self._perm]

    def combine(self, x: torch.Tensor, phase: int = 3) -> torch.Tensor:
        W, mm = self.world_size, self.max_m
        if phase != 2:
            # back to the receive layout, compacted source by source for the return trip
            slots = torch.zeros((W * mm, self.hidden), dtype=x.dtype, device=x.device)
            slots[self._perm] = x
            per_src = self._splits.view(W, self.epr).sum(1).tolist()
            self._back = torch.cat([slots[s * mm: s * mm + n] for s, n in enumerate(per_src)]) if sum(per_src) else slots[:0]
            self._back_cums = torch.zeros(self.num_experts + 1, dtype=torch.int32, device=x.device)
            self._back_cums[1:] = torch.cumsum(self._splits.reshape(-1), 0)
        _s, back, _ = A.fast_all_to_all(self.c_ctx, self._back.contiguous(), self._back_cums, None, phase=phase)
        if phase == 1:
            return None
        r = self._routing
        er = self._ids.reshape(-1).long() // self.epr
        row = er * mm + (r.slot_of.long() - r.cumsum.long()[er * self.epr])
        return back[row].float().view(self._ntok, self.topk, self.hidden).sum(1).to(x.dtype)


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
