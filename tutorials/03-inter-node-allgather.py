"""Tutorial 03 — the "inter-node" all-gather API on one NVSwitch node.

The reference's 2-D variants (``push_3d``, ``push_numa_2d``, ``..._multinode``) first move data between nodes
(or NUMA domains) and then fan it out locally. An 8xB200 box has ONE level: every GPU reaches every
other at full NVLink bandwidth through the switch. The mode names are kept so that code written against the
reference runs unchanged, and they map onto the single-level kernels; ``AllGatherLayer`` keeps the
reference's constructor (nnodes, world, rank, ...). (reference tutorials/03-inter-node-allgather.py,
layers/nvidia/low_latency_allgather_layer.py)
"""
import torch

from _common import dist_print, launch
from triton_distributed_b200.models import AllGatherLayer


def run(group, rank, world, dev):
    layer = AllGatherLayer(nnodes=1, world_size=world, rank=rank, max_buffer_size=1 << 20, group=group, device=dev)
    seg = torch.full((2048,), float(rank), dtype=torch.bfloat16, device=dev)
    want = torch.arange(world, device=dev).repeat_interleave(2048).to(torch.bfloat16)
    for name in ("forward_push_3d", "forward_push_numa_2d", "forward_push_numa_2d_ll_multinode", "forward_pull"):
        out = getattr(layer, name)(seg)
        assert torch.equal(out.reshape(-1), want), name
    dist_print("the 2-D / multi-node mode names all run the single-level kernels: ok")


if __name__ == "__main__":
    launch(run)
