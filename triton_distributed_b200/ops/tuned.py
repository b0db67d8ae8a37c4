"""Autotuned entry points: the hot ops wrapped as ``@tunable`` functions over the knobs their launchers expose.

Used inside a ``contextual_autotune`` thunk, every rank measures the same configuration at the same time and the
slowest rank's time decides, so all ranks settle on the same winner (reference python/triton_dist/autotuner.py:97-256;
its AG-GEMM test drives ``ag_gemm_intra_node`` this way, test/nvidia/test_ag_gemm_intra_node.py:112,200, over the
``triton.autotune`` space of kernels/nvidia/allgather_gemm.py:384-402). The kernels here are compiled ahead of time,
so the spaces are launch-time knobs: how the grid is split between pusher and GEMM CTAs, which tiling the GEMM
takes, how many KV splits the decode kernel uses, how many CTAs the MoE dispatch spreads over.

    @contextual_autotune(is_dist=True)
    def step():
        return ag_gemm_intra_node_tuned(a, w, ctx)

Outside a thunk the wrappers run the first configuration (the launchers' own heuristics).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..utils.autotuner import tunable
from . import flash_decode as FD
from . import gemm as G
from . import moe_ep as EP

# 0 / -1 = the launcher's own choice; the other points bracket it
AG_GEMM_SPACE = [{"num_comm_sms": c, "cta_pair": p} for p in (-1, 1, 2) for c in (0, 4, 8, 12, 16, 24)]
GEMM_RS_SPACE = [{"cta_pair": p} for p in (-1, 1, 2)]
DECODE_SPACE = [{"kv_split": s} for s in (-1, 4, 8, 16, 32, 64)]
MOE_DISPATCH_SPACE = [{"num_ctas": c} for c in (0, 32, 64, 148)]


@tunable(configs=AG_GEMM_SPACE, key=lambda a, b, ctx, out=None: (tuple(a.shape), tuple(b.shape), ctx.world), name="ag_gemm_intra_node")
def ag_gemm_intra_node_tuned(a: torch.Tensor, b: torch.Tensor, ctx, out: Optional[torch.Tensor] = None, *, config):
    saved = ctx.num_comm_sms, ctx.cta_pair
    ctx.num_comm_sms, ctx.cta_pair = config["num_comm_sms"], config["cta_pair"]
    try:
        return G.ag_gemm_intra_node(a, b, ctx, out=out)
    finally:
        ctx.num_comm_sms, ctx.cta_pair = saved


@tunable(configs=GEMM_RS_SPACE, key=lambda a, b, ctx, out=None: (tuple(a.shape), tuple(b.shape), ctx.world), name="gemm_rs")
def gemm_rs_tuned(a: torch.Tensor, b: torch.Tensor, ctx, out: Optional[torch.Tensor] = None, *, config):
    saved = ctx.cta_pair
    ctx.cta_pair = config["cta_pair"]
    try:
        return G.gemm_rs(a, b, ctx, out=out)
    finally:
        ctx.cta_pair = saved


@tunable(configs=DECODE_SPACE, key=lambda q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap=0.0: (
    tuple(q.shape), k_cache.shape[1], k_cache.shape[2], block_table.shape[1]), name="gqa_fwd_batch_decode")
def gqa_fwd_batch_decode_tuned(q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap: float = 0.0, *, config):
    return FD.gqa_fwd_batch_decode(q, k_cache, v_cache, None, None, kv_lens, block_table, scale, soft_cap,
                                   kv_split=config["kv_split"])


@tunable(configs=MOE_DISPATCH_SPACE, key=lambda ctx, x, topk_ids, topk_weights=None: (tuple(x.shape), ctx.world, ctx.num_experts),
         name="ep_dispatch")
def ep_dispatch_tuned(ctx, x, topk_ids, topk_weights=None, *, config):
    saved = ctx.num_ctas
    ctx.num_ctas = config["num_ctas"]
    try:
        return EP.ep_dispatch(ctx, x, topk_ids, topk_weights)
    finally:
        ctx.num_ctas = saved
