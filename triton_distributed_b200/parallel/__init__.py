"""Parallelism strategies the op library serves: tensor parallel (with Megatron-style sequence-parallel
activations), sequence-parallel long-context decode, expert parallel.

The reference has one flat group for everything (``TP_GROUP`` = all ranks, reference
python/triton_dist/utils.py:91-117) and no data or pipeline parallelism; its inter-node variants add a
(node, local rank) hierarchy. On one NVSwitch node the hierarchy is one level, so :class:`ParallelState`
carries a single group plus the node-shape queries the reference's APIs take as arguments.
"""
from .state import ParallelState, get_parallel_state, init_parallel_state
from .tensor_parallel import ColumnParallelLinear, RowParallelLinear, shard_columns, shard_rows
from .sequence_parallel import SequenceParallelKVCache, kv_lens_per_rank, shard_sequence
from .expert_parallel import ExpertPlacement, experts_of_rank

__all__ = [
    "ParallelState", "get_parallel_state", "init_parallel_state",
    "ColumnParallelLinear", "RowParallelLinear", "shard_columns", "shard_rows",
    "SequenceParallelKVCache", "kv_lens_per_rank", "shard_sequence",
    "ExpertPlacement", "experts_of_rank",
]
