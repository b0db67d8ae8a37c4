"""Expert parallelism: experts are split evenly and contiguously over the ranks; tokens travel to their
experts and back through the low-latency all-to-all (reference kernels/nvidia/low_latency_all_to_all.py:
189-248, layers/nvidia/ep_a2a_layer.py:187-206)."""
from __future__ import annotations

from dataclasses import dataclass

import torch


def experts_of_rank(num_experts: int, rank: int, world: int) -> range:
    per = num_experts // world
    return range(rank * per, (rank + 1) * per)


@dataclass
class ExpertPlacement:
    num_experts: int
    world: int

    def __post_init__(self):
        if self.num_experts % self.world:
            raise ValueError("the number of experts must be divisible by the world size")

    @property
    def experts_per_rank(self) -> int:
        return self.num_experts // self.world

    def owner(self, expert_ids: torch.Tensor) -> torch.Tensor:
        """Rank that hosts each expert id."""
        return expert_ids // self.experts_per_rank

    def local_index(self, expert_ids: torch.Tensor) -> torch.Tensor:
        return expert_ids % self.experts_per_rank

    def send_counts(self, topk_ids: torch.Tensor) -> torch.Tensor:
        """``[world, experts_per_rank]`` number of (token, k) pairs this rank sends to every expert."""
        return torch.bincount(topk_ids.reshape(-1).long(), minlength=self.num_experts).view(self.world, self.experts_per_rank)
