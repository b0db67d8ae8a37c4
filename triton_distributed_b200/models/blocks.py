"""Model blocks built from the fused ops: the units the end-to-end benchmark and the smoke test drive."""
from __future__ import annotations


import torch
import torch.nn.functional as F

from ..ops import gemm as G
from ..ops import moe_ep as EP
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
    """Expert-parallel MoE feed-forward: gate -> softmax top-k -> dispatch -> per-expert ``act(x W1^T) W2^T`` as two
    grouped tcgen05 GEMMs -> weighted combine. ``w1`` ``[E/ws, ffn, hidden]``, ``w2`` ``[E/ws, hidden, ffn]`` are this
    rank's experts; ``gate`` ``[E, hidden]`` is replicated.

    The dispatch kernel writes the received rows grouped by local expert with every group starting on a 128-row
    boundary, together with the expert of every 128-row block, so the receive buffer is the A operand of the
    grouped GEMM as it stands; the second GEMM writes into the symmetric buffer the combine kernels of the source
    ranks read. Five launches (top-k, dispatch, GEMM, activation, GEMM) + combine, no host synchronisation."""

    def __init__(self, gate: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk: int, rank: int, world: int, max_tokens: int,
                 group=None, heap=None):
        self.gate, self.w1, self.w2, self.topk, self.rank, self.world = gate, w1, w2, topk, rank, world
        self.E = gate.shape[0]
        self.epr = self.E // world
        self.hidden = gate.shape[1]
        self.ctx = EP.create_ep_context(max_tokens, self.hidden, topk, self.E, rank, world, quant=False, compact=True,
                                        align=MT.GROUP_BLOCK_M, heap=heap, group=group, device=gate.device)

    def experts(self, rows: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        """This rank's experts over the dispatched rows (``[capacity, hidden]``, block-aligned groups)."""
        h = MT.group_gemm(rows, self.w1, self.ctx.block_expert, self.ctx.num_blocks)
        return MT.group_gemm(F.silu(h), self.w2, self.ctx.block_expert, self.ctx.num_blocks, out=out)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = x.float() @ self.gate.float().t()
        ids, w = MU.topk_softmax(logits, self.topk, renormalize=True)
        rows, _, _, _ = EP.ep_dispatch(self.ctx, x, ids, w)
        if x.device.type != "cuda":
            return EP.ep_combine(self.ctx, self._experts_cpu(rows), weighted=True)
        self.experts(rows, out=EP.expert_out_buffer(self.ctx))
        return EP.ep_combine(self.ctx, None, weighted=True)

    def _experts_cpu(self, rows: torch.Tensor) -> torch.Tensor:
        # CPU ranks (gloo): the same block-aligned layout, block by block
        al = self.ctx.align
        counts = self.ctx.recv_splits.sum(0)
        out = torch.zeros_like(rows)
        off = 0
        for le in range(self.epr):
            n = int(counts[le])
            blk = slice(off, off + n)
            hmid = F.silu((rows[blk].float() @ self.w1[le].float().t()).to(rows.dtype))
            out[blk] = (hmid.float() @ self.w2[le].float().t()).to(rows.dtype)
            off += (n + al - 1) // al * al
        return out

    __call__ = forward
