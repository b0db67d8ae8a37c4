"""Tutorial 01 — notify / wait: a producer / consumer queue between neighbouring GPUs, written by hand.

The two primitives every overlapped kernel of this library is built from (``csrc/device/signal.cuh``):

    // producer (one thread, after the CTA's stores and a __syncthreads):
    tdist::notify(win, flag, peer, value, tdist::kSignalSet);    // fence.acq_rel.sys + st.release.sys on the peer
    // consumer (one warp):
    bool token = tdist::wait(flag, 1, value, wctx);              // bounded ld.acquire.sys spin
    data = tdist::consume_token(data, token);                    // + async-proxy fence if TMA reads the data next
    // and the address translation both use:
    float* remote = tdist::symm_at(win, local_ptr, peer);        // same offset in the peer's copy

``tutorials/kernels/notify_wait_queue.cu`` is a complete user kernel on top of them: rank r's producer CTAs stream
tiles into a ring of slots in rank r+1's symmetric memory, rank r+1's consumer CTAs drain it, and the ring is much
shorter than the stream, so each side keeps waiting for the other (slot "full" flags one way, "empty" flags back).
This script compiles that file against the library's headers, allocates the queue and the flags on the symmetric
heap, runs the kernel twice in a row without resetting anything (the flags only grow) and checks the result.

Every wait has a time limit: a flag that never comes makes the kernel record (kernel, rank, peer, site) in the
status block and return, instead of hanging the GPU. ``check_status()`` turns that record into an exception.
(reference tutorials/01-distributed-notify-wait.py: the same queue as a Triton kernel, 16 producer + 4 consumer CTAs)
"""
import ctypes as C
import os

import torch
import torch.distributed as dist

from _common import dist_print, launch

KERNEL = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernels", "notify_wait_queue.cu")


def run(group, rank, world, dev):
    n_tiles, tile, slots, producers, consumers = 96, 1024, 8, 8, 4
    gen = torch.Generator().manual_seed(1234)                       # every rank can rebuild everybody's input
    inputs = torch.randn(world, n_tiles, tile, generator=gen)
    left = (rank - 1) % world
    if dev.type != "cuda":
        # the same data flow with host send/recv, to show it on a machine without GPUs
        got = torch.empty(n_tiles, tile)
        if world > 1:
            for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, inputs[rank].contiguous(), (rank + 1) % world),
                                             dist.P2POp(dist.irecv, got, left)]):
                w.wait()
        else:
            got = inputs[rank]
        assert torch.equal(got, inputs[left])
        dist_print(f"[cpu] rank {rank} received the stream of rank {left}", allowed_ranks="all")
        return
    from triton_distributed_b200.runtime import check_status, default_timeout_ns, global_status, symm_heap
    from triton_distributed_b200.utils.user_kernels import load_user_library

    lib = load_user_library(KERNEL)                                  # nvcc -> tutorials/kernels/_build/, once
    lib.tutorial_queue_launch.restype = C.c_ulonglong
    lib.tutorial_queue_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                          C.c_int, C.c_int, C.c_int, C.c_ulonglong, C.c_void_p, C.c_ulonglong, C.c_void_p]
    heap = symm_heap(group)
    queue = heap.empty((slots, tile), torch.float32)                 # rank r+1's copy is what rank r writes into
    flags = heap.zeros((2 * slots,), torch.int64)                    # full[slots] then empty[slots]
    x = inputs[rank].to(dev)
    out = torch.empty_like(x)
    base = 0
    for call in range(2):
        if call == 1:
            x = x.flip(0).contiguous()                               # different data, same queue, no reset
        out.fill_(float("nan"))
        base = lib.tutorial_queue_launch(queue.ptr_array(), flags.ptr_array(), rank, world, x.data_ptr(), out.data_ptr(), n_tiles,
                                         tile, slots, producers, consumers, base, global_status().device_ptr, default_timeout_ns(),
                                         torch.cuda.current_stream().cuda_stream)
        assert base > 0, "bad launch arguments"
        torch.cuda.synchronize()
        check_status()                                               # raises if a wait ran out
        want = inputs[left].to(dev)
        torch.testing.assert_close(out, 2 * (want.flip(0) if call == 1 else want))
    if world > 1:
        dist.barrier(group)
    dist_print(f"rank {rank}: {n_tiles} tiles through an {slots}-slot queue from rank {left}, twice, ok", allowed_ranks="all")


if __name__ == "__main__":
    launch(run)
