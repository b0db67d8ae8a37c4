"""Tutorial 02 — intra-node all-gather, four ways.

The buffer is *symmetric*: every rank allocates the same object from the symmetric heap and can address
every peer's copy (``buf.peers[r]``). Rank r fills segment r of its own copy; afterwards every copy holds
all segments.

* ``pull``       signal "my segment is ready", then read every peer's segment over NVLink.
* ``push2d``     write my segment into every peer's copy, then raise my flag there.
* ``push2d_ll``  the same in 16-byte packets that carry their own flag: no separate signal, lowest latency
                 for small messages (twice the bytes on the wire).
* ``push2d_ll_multimem`` one ``multimem.st`` per 16 bytes stores into ALL copies through the NVSwitch
                 (needs ``TDIST_NVLS=1`` so that the heap binds a multicast object; else it runs as LL).

(reference tutorials/02-intra-node-allgather.py; kernels/nvidia/low_latency_allgather.py)
"""
import torch

from _common import dist_print, launch
from triton_distributed_b200.ops import collectives as CO
from triton_distributed_b200.runtime import symm_heap
from triton_distributed_b200.utils import perf_func


def run(group, rank, world, dev):
    heap = symm_heap(group)
    n = 8192 * world
    buf = heap.empty((n,), torch.int32)
    ctx = CO.create_fast_allgather_context(rank, 0, world, 1, max_buffer_size=n * 4, group=group, device=dev)
    want = torch.arange(world, dtype=torch.int32, device=dev).repeat_interleave(n // world)
    for mode in ("pull", "push2d", "push2d_ll", "push2d_ll_multimem"):
        buf.local.fill_(-1)
        buf.local[rank * (n // world):(rank + 1) * (n // world)] = rank
        heap.barrier()
        CO.fast_allgather(buf, ctx, mode=mode)
        if dev.type == "cuda":
            torch.cuda.synchronize()
        assert torch.equal(buf.local, want), mode
        heap.barrier()
        if dev.type == "cuda":
            def step():
                CO.fast_allgather(buf, ctx, mode=mode)
                CO.barrier_all_on_stream()
            _, ms = perf_func(step, 20, 5)
            dist_print(f"{mode:>20}: {ms * 1e3:7.1f} us per all-gather + barrier ({n * 4} bytes)")
    dist_print("all-gather ok in every mode")


if __name__ == "__main__":
    launch(run)
