"""Tutorial 05 — intra-node reduce-scatter.

Every rank holds a full ``[M, N]`` partial result; rank r needs the sum over ranks of rows
``[r*M/ws, (r+1)*M/ws)``. One kernel: each rank *pushes* the row block that belongs to peer p into p's staging
(slot = sender), raises its flag there, then waits for its own world-1 senders and adds their blocks to its
own in fp32. Staging is double-buffered by call parity. (reference tutorials/05-intra-node-reduce-scatter.py,
kernels/nvidia/reduce_scatter.py)
"""
import torch
import torch.distributed as dist

from _common import dist_print, launch
from triton_distributed_b200.ops import collectives as CO


def run(group, rank, world, dev):
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    M, N = 256 * world, 1024
    ctx = CO.create_reduce_scater_2d_ctx(M, N, rank, world, dtype=dtype, group=group, device=dev)
    for it in range(3):
        x = torch.randn(M, N, generator=torch.Generator().manual_seed(10 * it + rank)).to(dev, dtype)
        out = CO.reduce_scatter_2d_op(x, ctx)
        ref = x.float().clone()
        if world > 1:
            dist.all_reduce(ref, group=group)
        mine = ref[rank * (M // world):(rank + 1) * (M // world)]
        torch.testing.assert_close(out.float(), mine, atol=5e-2, rtol=2e-2)
    dist_print("reduce-scatter ok")


if __name__ == "__main__":
    launch(run)
