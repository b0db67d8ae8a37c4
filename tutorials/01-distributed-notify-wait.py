"""Tutorial 01 — notify / wait: the two primitives every overlapped kernel here is built from.

A producer writes data into a peer's symmetric buffer and then *notifies* a flag there; the consumer
*waits* on its own flag before it touches the data. In CUDA (``csrc/device/signal.cuh``):

    // producer (one thread, after the CTA's stores and a __syncthreads):
    tdist::notify(win, flag, peer, value, tdist::kSignalSet);    // fence.acq_rel.sys + st.release.sys on the peer
    // consumer (one warp):
    bool token = tdist::wait(flag, 1, value, wctx);              // bounded ld.acquire.sys spin
    data = tdist::consume_token(data, token);                    // + async-proxy fence if TMA reads the data next

Every wait has a time limit: a flag that never comes makes the kernel record (kernel, rank, peer, site) in
the status block and return, instead of hanging the GPU. ``check_status()`` turns that record into an
exception on the host.

This script runs the ring version of the protocol on every rank: rank r puts a block into rank r+1 and
notifies it; everybody waits for its left neighbour. (reference tutorials/01-distributed-notify-wait.py)
"""
import torch
import torch.distributed as dist

from _common import dist_print, launch


def run(group, rank, world, dev):
    if dev.type != "cuda":
        # the same protocol with host send/recv, to show the data flow on a machine without GPUs
        token = torch.full((4,), float(rank))
        got = torch.empty(4)
        ops = [dist.P2POp(dist.isend, token, (rank + 1) % world), dist.P2POp(dist.irecv, got, (rank - 1) % world)] if world > 1 else []
        for w in (dist.batch_isend_irecv(ops) if ops else []):
            w.wait()
        if world > 1:
            assert got[0].item() == (rank - 1) % world
        dist_print(f"[cpu] rank {rank} received the block of rank {(rank - 1) % world}", allowed_ranks="all")
        return
    from triton_distributed_b200.ops import primitives as P
    from triton_distributed_b200.runtime import check_status
    ctx = P.create_primitive_context(rank, world, nbytes=4096, group=group)
    ctx.source.copy_(torch.full((4096,), rank + 1, dtype=torch.uint8, device=dev))
    torch.cuda.synchronize()
    dist.barrier(group)
    left = (rank - 1) % world
    for it in range(1, 4):
        # putmem_signal: copy my block into rank+1's slot `rank`, then set its signal word to `it`; my own kernel
        # then waits until MY signal word has been set by rank-1 and reports whether the wait succeeded
        P.run_primitive(ctx, "put_signal", value=it, scope="block")
        torch.cuda.synchronize()
        check_status()                                    # raises if a wait ran out
        assert int(ctx.result[0]) == 1
        assert int(ctx.slot(left)[0]) == left + 1 and int(ctx.slot(left)[-1]) == left + 1
        # This demo kernel waits for EQUALITY with `it`, so no rank may run a round ahead: keep them in step. (The
        # fused ops avoid the host barrier by waiting for >= a call number that only grows.)
        dist.barrier(group)
    dist_print(f"rank {rank}: putmem_signal ring + bounded wait ok", allowed_ranks="all")


if __name__ == "__main__":
    launch(run)
