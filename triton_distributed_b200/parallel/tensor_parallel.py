"""Tensor parallelism with sequence-parallel activations (the Megatron pairing):

* :class:`ColumnParallelLinear` — activations arrive row(token)-sharded, weights are column-sharded:
  ``y[M, N/ws] = allgather(x[M/ws, K]) @ W[N/ws, K]^T`` = one fused AG-GEMM launch.
* :class:`RowParallelLinear` — activations are column-sharded, the output leaves row-sharded:
  ``y[M/ws, N] = reduce_scatter(x[M, K/ws] @ W[N, K/ws]^T)`` = one fused GEMM-RS launch.

(reference kernels/nvidia/allgather_gemm.py:785-882 and gemm_reduce_scatter.py:482-538 are the two ops;
the reference leaves the layer pairing to its tests, test/nvidia/test_ag_gemm_intra_node.py and
test_gemm_rs.py.)
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import gemm as G
from ..ops import gemm_fp8 as F8
from .state import ParallelState, get_parallel_state


def shard_rows(full: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows ``[rank*M/ws, (rank+1)*M/ws)`` of ``full`` (a contiguous copy)."""
    per = full.shape[0] // world
    return full[rank * per:(rank + 1) * per].contiguous()


def shard_columns(full: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Columns ``[rank*K/ws, (rank+1)*K/ws)`` of ``full`` (a contiguous copy)."""
    per = full.shape[1] // world
    return full[:, rank * per:(rank + 1) * per].contiguous()


class ColumnParallelLinear:
    """``weight`` is this rank's ``[N/ws, K]`` shard. ``fp8=True`` quantises the weight once to e4m3 with
    128 x 128 block scales and each call's activations to 1 x 128 scales, and runs the fp8 AG-GEMM."""

    def __init__(self, weight: torch.Tensor, max_tokens: int, state: Optional[ParallelState] = None, heap=None, fp8: bool = False):
        self.state = state or get_parallel_state()
        s = self.state
        self.fp8 = fp8
        if fp8:
            self.weight, self.weight_scale = F8.quantize_fp8_blockwise(weight)
            self.ctx = F8.create_ag_gemm_fp8_context(max_tokens, weight.shape[1], s.rank, s.world, device=weight.device,
                                                     heap=heap, group=s.group)
        else:
            self.weight = weight.contiguous()
            proto = torch.empty((1, weight.shape[1]), dtype=weight.dtype, device=weight.device)
            self.ctx = G.create_ag_gemm_intra_node_context(proto, self.weight, s.rank, s.world, max_M=max_tokens, group=s.group, heap=heap)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        if self.fp8:
            a, sa = F8.quantize_fp8_rowwise(x_shard)
            return F8.ag_gemm_fp8(a, sa, self.weight, self.weight_scale, self.ctx)
        return G.ag_gemm_intra_node(x_shard, self.weight, self.ctx)

    __call__ = forward


class RowParallelLinear:
    """``weight`` is this rank's ``[N, K/ws]`` shard; the result is this rank's ``[M/ws, N]`` rows."""

    def __init__(self, weight: torch.Tensor, max_tokens: int, state: Optional[ParallelState] = None, heap=None):
        self.state = state or get_parallel_state()
        s = self.state
        self.weight = weight.contiguous()
        self.ctx = G.create_gemm_rs_context(max_tokens, weight.shape[0], s.rank, s.world, output_dtype=weight.dtype,
                                            group=s.group, heap=heap, device=weight.device)

    def forward(self, x_cols: torch.Tensor) -> torch.Tensor:
        return G.gemm_rs(x_cols, self.weight, self.ctx)

    __call__ = forward
