"""Tutorial 06 — reduce-scatter and all-reduce *inside the switch* (NVLS).

The reference's tutorial 06 reduces across nodes in two stages. One NVSwitch node has a better tool: bind
every rank's copy of a symmetric buffer to one multicast object and let the switch do the arithmetic.

    multimem.ld_reduce.add  [mc + x]   -> the sum of all ranks' values at offset x, added in the switch
    multimem.st             [mc + x]   -> stores into every rank's copy

``nvls_reduce_scatter``: rank r reads the reduced segment r. ``nvls_allreduce``: rank r reduces segment r and
multicasts it back, in place — each byte crosses each link once in each direction.

Run with ``TDIST_NVLS=1`` so that the heap binds a multicast object; without it (or on CPU) the script shows
the API on the fallback paths. (reference tutorials/06-inter-node-reduce-scatter.py)
"""
import torch
import torch.distributed as dist

from _common import dist_print, launch
from triton_distributed_b200.ops import collectives as CO
from triton_distributed_b200.ops import nvls as NV
from triton_distributed_b200.runtime import symm_heap


def run(group, rank, world, dev):
    heap = symm_heap(group)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    n = 64 * 1024 * world
    buf = heap.empty((n,), dtype)
    x = torch.randn(n, generator=torch.Generator().manual_seed(rank)).to(dev, dtype)
    ref = x.float().clone()
    if world > 1:
        dist.all_reduce(ref, group=group)
    seg = n // world
    if dev.type == "cuda" and world > 1 and not NV.nvls_available(buf):
        dist_print("no multicast alias (set TDIST_NVLS=1 on an NVSwitch system): using the push reduce-scatter instead")
        ctx = CO.create_reduce_scater_2d_ctx(world, seg, rank, world, dtype=dtype, group=group, device=dev)
        out = CO.reduce_scatter_2d_op(x.view(world, seg), ctx)
        torch.testing.assert_close(out.float().view(-1), ref[rank * seg:(rank + 1) * seg], atol=5e-2, rtol=2e-2)
        return
    ctx = NV.create_nvls_context(rank, world, heap=heap, group=group, device=dev)
    buf.local.copy_(x)
    heap.barrier()
    out = NV.nvls_reduce_scatter(buf, ctx)
    torch.testing.assert_close(out.float(), ref[rank * seg:(rank + 1) * seg], atol=5e-2, rtol=2e-2)
    heap.barrier()
    NV.nvls_allreduce(buf, ctx)
    torch.testing.assert_close(buf.local.float(), ref, atol=5e-2, rtol=2e-2)
    dist_print("switch-side reduce-scatter and all-reduce ok")


if __name__ == "__main__":
    launch(run)
