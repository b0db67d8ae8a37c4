"""Shared launcher of the tutorials: one process per GPU under torchrun (NCCL), or gloo ranks on CPU.

    torchrun --nproc-per-node 8 tutorials/07-overlapping-allgather-gemm.py
    CUDA_VISIBLE_DEVICES= torchrun --nproc-per-node 2 tutorials/07-overlapping-allgather-gemm.py   # CPU restatement
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from triton_distributed_b200.runtime import finalize_distributed, initialize_distributed  # noqa: E402
from triton_distributed_b200.utils import dist_print  # noqa: E402,F401


def launch(run):
    """Initialise torch.distributed + the symmetric heap, call ``run(group, rank, world, device)``, tear down."""
    if "RANK" not in os.environ:  # plain `python tutorial.py` = a world of one
        os.environ.update({"RANK": "0", "LOCAL_RANK": "0", "WORLD_SIZE": "1", "MASTER_ADDR": "127.0.0.1",
                           "MASTER_PORT": os.environ.get("MASTER_PORT", "29533")})
    group = initialize_distributed(seed=0)
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    try:
        run(group, rank, world, dev)
    finally:
        finalize_distributed()
