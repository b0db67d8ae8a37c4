"""Process-group bootstrap: one process per GPU, ``torchrun`` environment.

Counterpart of the reference's ``initialize_distributed`` / ``TP_GROUP``
(reference python/triton_dist/utils.py:75-117), which also brings up NVSHMEM; here the
symmetric heap is created lazily by :func:`symm_heap` on first use.
"""
from __future__ import annotations

import datetime
import os
import random
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from .heap import SymmetricHeap

_TP_GROUP = None
_HEAP: Optional[SymmetricHeap] = None


def init_seed(seed: int = 0) -> None:
    """Deterministic seeding of torch / numpy / random (reference utils.py:75-88)."""
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    np.random.seed(seed)
    random.seed(seed)


def initialize_distributed(backend: Optional[str] = None, seed: Optional[int] = None, timeout_s: int = 1800):
    """Initialise ``torch.distributed`` from RANK / LOCAL_RANK / WORLD_SIZE and return the group of
    all ranks. Uses NCCL when a GPU is present, gloo otherwise."""
    global _TP_GROUP
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    if use_cuda:
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        kwargs = dict(backend=backend, world_size=world, rank=rank, timeout=datetime.timedelta(seconds=timeout_s))
        if use_cuda and backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(**kwargs)
    _TP_GROUP = dist.new_group(ranks=list(range(world)), backend=backend)
    init_seed(rank if seed is None else seed)
    return _TP_GROUP


def TP_GROUP():
    """The group created by :func:`initialize_distributed` (all ranks)."""
    if _TP_GROUP is None:
        raise RuntimeError("initialize_distributed() has not been called")
    return _TP_GROUP


def symm_heap(group=None) -> SymmetricHeap:
    """Process-wide symmetric heap over ``group`` (default: the TP group), created on first use."""
    global _HEAP
    if _HEAP is None:
        if group is None and _TP_GROUP is not None:
            group = _TP_GROUP
        _HEAP = SymmetricHeap(group)
    return _HEAP


def set_symm_heap(heap) -> None:
    """Install ``heap`` (e.g. a LocalWorld rank view) as the process-wide heap."""
    global _HEAP
    _HEAP = heap


def finalize_distributed() -> None:
    """Unmap the symmetric heap and destroy the process group."""
    global _HEAP, _TP_GROUP
    if _HEAP is not None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
        _HEAP.close()
        _HEAP = None
    if dist.is_initialized():
        dist.destroy_process_group()
    _TP_GROUP = None
