"""MoE routing utilities: softmax/top-k selection, expert-sorted permutation, block-aligned sort.

* ``topk_softmax(logits, topk)`` — gate probabilities and expert ids per token
  (reference ``select_experts``: kernels/nvidia/moe_reduce_rs.py:180-197 does this with torch ops).
* ``route(topk_ids, num_experts)`` — splits / cumsum / sorted order of the (token, k) pairs, what the
  reference assembles from ``torch.bincount`` + ``argsort`` + ``kernel_bincount``
  (kernels/nvidia/ep_a2a.py:309-335, test/nvidia/test_all_to_all.py ``calc_gather_index``).
* ``sort_topk_ids_align_block_size`` — rank-major, block-padded expert sort for the MoE group GEMMs
  (reference kernels/nvidia/allgather_group_gemm.py:54-137 calling csrc/lib/moe_utils.cu).
* ``full_moe_align_block_size`` — slow, obviously-correct torch restatement used as the oracle
  (reference kernels/nvidia/moe_reduce_rs.py:87-177).

CUDA tensors run the kernels in ``csrc/kernels/moe.cu``; CPU tensors run the torch restatements.
"""
from __future__ import annotations

from typing import NamedTuple, Optional, Tuple

import torch

from .. import _lib

launch_count = 0


def _stream(t: torch.Tensor, stream=None):
    return (stream or torch.cuda.current_stream(t.device)).cuda_stream


def _status_ptr():
    from ..runtime.status import global_status
    st = global_status()
    return st.device_ptr if st is not None else None


class Routing(NamedTuple):
    splits: torch.Tensor        # int32 [E]   pairs per expert
    cumsum: torch.Tensor        # int32 [E+1] exclusive prefix sum
    sorted_token: torch.Tensor  # int32 [n]   token of the pair at each expert-sorted position
    slot_of: torch.Tensor       # int32 [n]   expert-sorted position of pair (t, k) (index t*topk+k)


def topk_softmax(logits: torch.Tensor, topk: int, renormalize: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``softmax(logits)`` over experts, then the ``topk`` largest per token.
    Returns ``(ids int32 [T, topk], weights fp32 [T, topk])``; ties go to the lower expert id."""
    global launch_count
    T, E = logits.shape
    if logits.device.type != "cuda":
        probs = torch.softmax(logits.float(), dim=-1)
        # stable descending sort = ties to the lower index, like the kernel
        order = torch.sort(probs, dim=-1, descending=True, stable=True)
        w, ids = order.values[:, :topk], order.indices[:, :topk]
        if renormalize:
            w = w / w.sum(-1, keepdim=True)
        return ids.to(torch.int32), w.contiguous()
    x = logits.float().contiguous()
    ids = torch.empty((T, topk), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, topk), dtype=torch.float32, device=logits.device)
    _lib.check(_lib.lib().tdist_moe_topk_softmax(x.data_ptr(), T, E, topk, int(renormalize), ids.data_ptr(),
                                                 w.data_ptr(), _stream(x)), "tdist_moe_topk_softmax")
    launch_count += 1
    return ids, w


def route(topk_ids: torch.Tensor, num_experts: int, out: Optional[Routing] = None) -> Routing:
    """Stable expert sort of the ``T*topk`` (token, k) pairs.

    An id outside ``[0, num_experts)`` (``-1`` for a dropped pair) is not counted and not sorted: its ``slot_of`` is
    ``-1``, and on CUDA the first such id is recorded as a bad argument in the status block, which
    ``check_status()`` raises."""
    global launch_count
    T, K = topk_ids.shape
    n = T * K
    dev = topk_ids.device
    if out is None:
        out = Routing(torch.empty(num_experts, dtype=torch.int32, device=dev),
                      torch.empty(num_experts + 1, dtype=torch.int32, device=dev),
                      torch.empty(n, dtype=torch.int32, device=dev), torch.empty(n, dtype=torch.int32, device=dev))
    if dev.type != "cuda":
        flat = topk_ids.reshape(-1).long()
        ok = (flat >= 0) & (flat < num_experts)
        key = torch.where(ok, flat, torch.full_like(flat, num_experts))      # rejected ids sort last
        splits = torch.bincount(key, minlength=num_experts + 1)[:num_experts]
        order = torch.sort(key, stable=True).indices
        live = int(ok.sum())
        out.splits.copy_(splits)
        out.cumsum[0] = 0
        out.cumsum[1:].copy_(torch.cumsum(splits, 0))
        out.sorted_token[:live].copy_(order[:live] // K)
        out.slot_of.fill_(-1)
        out.slot_of[order[:live]] = torch.arange(live, dtype=torch.int32)
        return out
    ids = topk_ids.contiguous()
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    _lib.check(_lib.lib().tdist_moe_route(ids.data_ptr(), n, K, num_experts, out.splits.data_ptr(), out.cumsum.data_ptr(),
                                          out.sorted_token.data_ptr(), out.slot_of.data_ptr(), _status_ptr(), _stream(ids)),
               "tdist_moe_route")
    launch_count += 1
    return out


def _align_capacities(numel_per_rank: int, num_experts: int, num_ranks: int, block_size: int) -> Tuple[int, int]:
    sorted_cap = (numel_per_rank + num_experts * (block_size - 1)) * num_ranks
    blocks_cap = (numel_per_rank + num_experts) * num_ranks
    return sorted_cap, blocks_cap


def sort_topk_ids_align_block_size(topk_ids: torch.Tensor, num_experts: int, num_ranks: int, num_tokens_per_rank: int,
                                   block_size: int, moe_stream=None):
    """Sort the pairs of all ranks' tokens rank by rank, expert by expert inside a rank, padding
    every (rank, expert) group to a multiple of ``block_size``.

    Returns ``(sorted_token_ids, expert_ids, block_barrier_ids, rank_block_num, num_tokens_post_pad)``:
    ``sorted_token_ids`` holds flattened pair indices (padding = ``topk_ids.numel()``),
    ``expert_ids[b]`` / ``block_barrier_ids[b]`` the expert and the source rank of block ``b``,
    ``rank_block_num[r]`` the number of blocks of rank ``r``."""
    global launch_count
    if topk_ids.device.type != "cuda":
        return full_moe_align_block_size(topk_ids, block_size, num_experts, num_ranks, num_tokens_per_rank)
    K = topk_ids.shape[1]
    numel = num_tokens_per_rank * K
    assert topk_ids.shape[0] == num_tokens_per_rank * num_ranks
    dev = topk_ids.device
    sorted_cap, blocks_cap = _align_capacities(numel, num_experts, num_ranks, block_size)
    sorted_ids = torch.empty(sorted_cap, dtype=torch.int32, device=dev)
    expert_ids = torch.zeros(blocks_cap, dtype=torch.int32, device=dev)
    barrier_ids = torch.zeros(blocks_cap, dtype=torch.int32, device=dev)
    rank_block_num = torch.empty(num_ranks, dtype=torch.int32, device=dev)
    post_pad = torch.empty(1, dtype=torch.int32, device=dev)
    ids = topk_ids.contiguous()
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    _lib.check(_lib.lib().tdist_moe_align_block_size(ids.data_ptr(), numel, num_experts, num_ranks, block_size,
                                                     sorted_ids.data_ptr(), sorted_cap, expert_ids.data_ptr(),
                                                     barrier_ids.data_ptr(), rank_block_num.data_ptr(),
                                                     post_pad.data_ptr(), _status_ptr(), _stream(ids, moe_stream)),
               "tdist_moe_align_block_size")
    launch_count += 1
    return sorted_ids, expert_ids, barrier_ids, rank_block_num, post_pad


def full_moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int, num_ranks: int,
                              num_tokens_per_rank: int):
    """Vectorised torch statement of the same layout (the oracle of the kernel)."""
    K = topk_ids.shape[1]
    numel = num_tokens_per_rank * K
    dev = topk_ids.device
    sorted_cap, blocks_cap = _align_capacities(numel, num_experts, num_ranks, block_size)
    sorted_ids = torch.full((sorted_cap,), topk_ids.numel(), dtype=torch.int32, device=dev)
    expert_ids = torch.zeros(blocks_cap, dtype=torch.int32, device=dev)
    barrier_ids = torch.zeros(blocks_cap, dtype=torch.int32, device=dev)
    rank_block_num = torch.empty(num_ranks, dtype=torch.int32, device=dev)
    flat = topk_ids.reshape(-1).long()
    base = 0
    for r in range(num_ranks):
        ids = flat[r * numel:(r + 1) * numel]
        counts = torch.bincount(ids, minlength=num_experts)
        padded = (counts + block_size - 1) // block_size * block_size
        starts = torch.cumsum(padded, 0) - padded
        order = torch.sort(ids, stable=True).indices
        sorted_e = ids[order]
        first_of_e = torch.cumsum(counts, 0) - counts
        pos = starts[sorted_e] + (torch.arange(numel, device=dev) - first_of_e[sorted_e])
        sorted_ids[base + pos] = (order + r * numel).to(torch.int32)
        nblocks = padded // block_size
        total_blocks = int(nblocks.sum())
        expert_ids[base // block_size: base // block_size + total_blocks] = torch.repeat_interleave(
            torch.arange(num_experts, device=dev, dtype=torch.int32), nblocks)
        barrier_ids[base // block_size: base // block_size + total_blocks] = r
        rank_block_num[r] = total_blocks
        base += int(padded.sum())
    post_pad = torch.tensor([base], dtype=torch.int32, device=dev)
    return sorted_ids, expert_ids, barrier_ids, rank_block_num, post_pad


def bincount(exp_indices: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Tokens per expert, int32 ``[num_experts]`` (reference kernels/nvidia/ep_a2a.py:309-321 ``kernel_bincount``): the
    ``splits`` of :func:`route`."""
    ids = exp_indices.reshape(-1, 1)
    return route(ids, num_experts).splits


def calc_gather_index(topk_ids: torch.Tensor, num_experts: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(gather_index, scatter_index)`` of the expert-sorted layout: row ``i`` of the sorted activations is token
    ``gather_index[i]``, and pair ``(t, k)`` sits at row ``scatter_index[t * topk + k]`` (the reference builds these
    with torch argsort in its MoE tests, test/nvidia/test_ag_moe.py)."""
    r = route(topk_ids, num_experts)
    return r.sorted_token, r.slot_of
