"""Process-group state shared by the strategies."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelState:
    """One flat group used as TP, SP and EP group alike (as in the reference), with the node shape.

    ``local_world`` / ``nnodes`` exist because the reference's contexts take them; every op here runs the
    single-level NVSwitch path, so ``nnodes`` must be 1 for the fused CUDA kernels (the CPU / gloo
    restatements accept any shape)."""

    group: object
    rank: int
    world: int
    local_rank: int
    local_world: int

    @property
    def nnodes(self) -> int:
        return max(1, self.world // max(1, self.local_world))

    @property
    def node(self) -> int:
        return self.rank // max(1, self.local_world)

    @property
    def is_single_node(self) -> bool:
        return self.nnodes == 1

    def device(self) -> torch.device:
        if torch.cuda.is_available():
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")


_STATE: Optional[ParallelState] = None


def init_parallel_state(group=None) -> ParallelState:
    """Build the state from an initialised ``torch.distributed`` (or a single process)."""
    global _STATE
    if dist.is_available() and dist.is_initialized():
        rank, world = dist.get_rank(group), dist.get_world_size(group)
    else:
        rank, world = 0, 1
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", world))
    local_rank = int(os.environ.get("LOCAL_RANK", rank % max(1, local_world)))
    _STATE = ParallelState(group=group, rank=rank, world=world, local_rank=local_rank, local_world=local_world)
    return _STATE


def get_parallel_state() -> ParallelState:
    return _STATE if _STATE is not None else init_parallel_state()
