"""Model blocks built from the fused ops: the units the end-to-end benchmark and the smoke test drive."""
from __future__ import annotations


import torch
import torch.nn.functional as F

from ..ops import all_to_all as A
from ..ops import gemm as G
from ..ops import moe_tp as MT
from ..ops import moe_utils as MU


class TPMLP:
    """Megatron-style tensor/sequence-parallel MLP over ``world`` ranks:
    ``y = reduce_scatter(act(allgather(x) @ W1_shard^T) @ W2_shard^T)``. ``x`` is this rank's
    ``[M/ws, hidden]`` token shard, ``w1`` ``[ffn/ws, hidden]``, ``w2`` ``[hidden, ffn/ws]``; the output
    is this rank's ``[M/ws, hidden]`` rows. Two kernel launches: AG-GEMM and GEMM-RS (+ activation)."""

    def __init__(self, w1: torch.Tensor, w2: torch.Tensor, rank: int, world: int, max_M: int, activation: str = "gelu",
                 group=None, heap=None):
        self.w1, self.w2, self.rank, self.world = w1, w2, rank, world
        self.activation = activation
        proto = torch.empty((1, w1.shape[1]), dtype=w1.dtype, device=w1.device)
        self.ag_ctx = G.create_ag_gemm_intra_node_context(proto, w1, rank, world, max_M=max_M, group=group, heap=heap)
        self.rs_ctx = G.create_gemm_rs_context(max_M, w2.shape[0], rank, world, output_dtype=w1.dtype, group=group, heap=heap,
                                               device=w1.device)

    def _act(self, h: torch.Tensor) -> torch.Tensor:
        if self.activation == "gelu":
            return F.gelu(h, approximate="tanh")
        if self.activation == "silu":
            return F.silu(h)
        if self.activation == "relu":
            return F.relu(h)
        return h

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = G.ag_gemm_intra_node(x, self.w1, self.ag_ctx)
        return G.gemm_rs(self._act(h), self.w2, self.rs_ctx)

    __call__ = forward


class EPMoE:
    """Expert-parallel MoE feed-forward: route -> fp8 dispatch -> per-expert ``act(x W1^T) W2^T`` as two
    grouped tcgen05 GEMMs over the received rows -> weighted combine. ``w1`` ``[E/ws, ffn, hidden]``,
    ``w2`` ``[E/ws, hidden, ffn]`` are this rank's experts; ``gate`` ``[E, hidden]`` is replicated."""

    def __init__(self, gate: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk: int, rank: int, world: int, max_tokens: int,
                 group=None, heap=None):
        self.gate, self.w1, self.w2, self.topk, self.rank, self.world = gate, w1, w2, topk, rank, world
        self.E = gate.shape[0]
        self.epr = self.E // world
        self.hidden = gate.shape[1]
        self.ctx = A.create_moe_dispatch_context(max_tokens, self.hidden, topk, self.E, rank, world, heap=heap, group=group,
                                                 device=gate.device)

    def experts(self, rx: torch.Tensor, rs: torch.Tensor, splits: torch.Tensor) -> torch.Tensor:
        """Run this rank's experts over the receive layout ``[ws*max_m, hidden]`` (rows of source s sorted
        by local expert inside slot s) and return outputs in the same layout."""
        W, mm = self.world, self.ctx.dispatch.max_m
        x = A.dequant_fp8(rx, rs)
        # every (source, local expert) run of rows is one group; pad groups to 128 rows for the grouped GEMM
        sp = splits.reshape(W, self.epr)
        ids = torch.full((W * mm,), -1, dtype=torch.int32, device=x.device)
        live_rows, expert_of_row = [], []
        counts = sp.tolist()
        for s in range(W):
            off = s * mm
            for e in range(self.epr):
                n = counts[s][e]
                if n:
                    live_rows.append(torch.arange(off, off + n, device=x.device))
                    expert_of_row.append(torch.full((n,), e, dtype=torch.int32, device=x.device))
                    off += n
        if not live_rows:
            return torch.zeros_like(x)
        rows = torch.cat(live_rows)
        eids = torch.cat(expert_of_row).view(-1, 1)
        sorted_ids, expert_ids, _, _, post_pad = MU.sort_topk_ids_align_block_size(eids, self.epr, 1, eids.shape[0], 128)
        n = int(post_pad)
        index = sorted_ids[:n].clone()
        live = index < rows.shape[0]
        index[live] = rows[index[live].long()].to(torch.int32)
        index[~live] = -1
        a_sorted, _ = MT.gather_rows(x, index, 1, W * mm)
        nb = (post_pad // 128).to(torch.int32)
        h = MT.group_gemm(a_sorted, self.w1, expert_ids, nb)
        h = F.silu(h)
        y_sorted = MT.group_gemm(h, self.w2, expert_ids, nb)
        out = torch.zeros_like(x)
        out[index[live].long()] = y_sorted[live]
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = x.float() @ self.gate.float().t()
        ids, w = MU.topk_softmax(logits, self.topk, renormalize=True)
        rx, rs, splits = A.moe_dispatch(self.ctx, x, ids, w)
        y = self.experts(rx, rs, splits)
        return A.moe_combine(self.ctx, y, splits)

    __call__ = forward
