"""Sequence parallelism for long-context decode: the KV cache of every sequence is cut along the
sequence into ``world`` contiguous shards; each rank attends its shard and the partial results are merged
by log-sum-exp inside the fused decode kernel (reference layers/nvidia/sp_flash_decode_layer.py:78-184).
The reference has no ring attention, Ulysses or prefill-side context parallelism, and neither has this.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch


def shard_sequence(global_len: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Keys of each sequence that fall into rank ``rank``'s shard when a sequence of ``global_len`` keys is
    cut into ``world`` contiguous shards of ``ceil(len / world)`` keys (the last shards may be short or empty)."""
    per = (global_len + world - 1) // world
    return (global_len - per * rank).clamp(min=0).minimum(per)


def kv_lens_per_rank(global_len: torch.Tensor, world: int) -> torch.Tensor:
    """``[world, B]`` keys held by every rank: the ``global_kv_lens`` argument of
    ``sp_gqa_fwd_batch_decode`` / ``SpGQAFlashDecodeAttention.forward``."""
    return torch.stack([shard_sequence(global_len, r, world) for r in range(world)]).to(torch.int32)


@dataclass
class SequenceParallelKVCache:
    """A paged KV cache holding this rank's shard: ``k`` / ``v`` are ``[pages, page_size, Hkv, D]``,
    ``block_table`` ``[B, max_pages]`` maps a sequence's local page number to a page."""

    k: torch.Tensor
    v: torch.Tensor
    block_table: torch.Tensor
    page_size: int
    rank: int
    world: int

    @classmethod
    def allocate(cls, batch: int, max_global_len: int, num_kv_heads: int, head_dim: int, rank: int, world: int,
                 page_size: int = 16, dtype=torch.bfloat16, device="cuda") -> "SequenceParallelKVCache":
        per = (max_global_len + world - 1) // world
        pages_per_seq = (per + page_size - 1) // page_size
        k = torch.zeros((batch * pages_per_seq, page_size, num_kv_heads, head_dim), dtype=dtype, device=device)
        v = torch.zeros_like(k)
        table = torch.arange(batch * pages_per_seq, dtype=torch.int32, device=device).view(batch, pages_per_seq)
        return cls(k, v, table, page_size, rank, world)

    def local_lens(self, global_lens: torch.Tensor) -> torch.Tensor:
        return shard_sequence(global_lens, self.rank, self.world)

    def write(self, seq: int, k_new: torch.Tensor, v_new: torch.Tensor, global_pos: int, global_len_after: int) -> bool:
        """Store the key/value of global position ``global_pos`` of sequence ``seq`` if it belongs to this
        rank's shard once the sequence has ``global_len_after`` keys. Shards are contiguous, so appending a
        token can move shard boundaries; serving systems therefore fix ``ceil(max_len / world)`` up front and
        this helper assumes ``global_len_after`` is that fixed maximum."""
        per = (global_len_after + self.world - 1) // self.world
        owner, local = divmod(global_pos, per)
        if owner != self.rank:
            return False
        page = int(self.block_table[seq, local // self.page_size])
        self.k[page, local % self.page_size].copy_(k_new)
        self.v[page, local % self.page_size].copy_(v_new)
        return True

    def shapes(self) -> Tuple[int, int, int, int]:
        return tuple(self.k.shape)
