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

The last part of the script does the push variant once more with a kernel written against the OpenSHMEM-style device
API of ``csrc/device/shmem.cuh`` (``tutorials/kernels/allgather_putmem_signal.cu``: ``putmem_signal_block`` into every
peer, then ``signal_wait_until`` on this rank's own signal words), compiled here with
``triton_distributed_b200.utils.user_kernels``: what a user of the primitives writes.

(reference tutorials/02-intra-node-allgather.py; kernels/nvidia/low_latency_allgather.py)
"""
import ctypes as C
import os

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
    if dev.type == "cuda":
        user_kernel_allgather(heap, rank, world, dev)
    dist_print("all-gather ok in every mode")


def user_kernel_allgather(heap, rank, world, dev):
    """The push all-gather as a user kernel on the shmem.cuh API: three calls on the same buffers, no reset between them
    (the signal words carry the call number)."""
    from triton_distributed_b200.runtime import check_status, default_timeout_ns, global_status
    from triton_distributed_b200.utils.user_kernels import load_user_library

    lib = load_user_library(os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernels", "allgather_putmem_signal.cu"))
    lib.tutorial_allgather_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_ulonglong, C.c_ulonglong, C.c_void_p,
                                              C.c_ulonglong, C.c_void_p]
    seg = 64 * 1024
    buf = heap.empty((world, seg), torch.uint8)
    sig = heap.zeros((world,), torch.int64)
    for call in range(1, 4):
        buf.local.fill_(255)
        buf.local[rank].fill_((rank * 7 + call) % 251)
        heap.barrier()                    # demo only: nobody's segment is overwritten by the fill above after it was pushed
        rc = lib.tutorial_allgather_launch(buf.ptr_array(), sig.ptr_array(), rank, world, seg, call, global_status().device_ptr,
                                           default_timeout_ns(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        check_status()
        want = torch.tensor([(r * 7 + call) % 251 for r in range(world)], dtype=torch.uint8, device=dev)
        assert torch.equal(buf.local, want.view(world, 1).expand(world, seg)), f"user-kernel all-gather, call {call}"
        heap.barrier()
    dist_print("putmem_signal_block / signal_wait_until all-gather (user kernel) ok")


if __name__ == "__main__":
    launch(run)
