"""Multi-rank check of barrier / all-gather / reduce-scatter (NCCL or gloo as oracle), with
random per-rank delays before each call (the reference's test_common_ops.py jitter idiom)."""
import json
import random

import torch
import torch.distributed as dist

from triton_distributed_b200.ops import collectives as CO
from triton_distributed_b200.runtime import check_status, finalize_distributed, initialize_distributed, symm_heap


def main():
    group = initialize_distributed(seed=0)
    rank, world = dist.get_rank(), dist.get_world_size()
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    res = {"world": world, "device": dev.type}
    rng = random.Random(rank)
    heap = symm_heap(group)

    # ---- barrier: a rank that is late must hold everybody back (GPU only; CPU uses dist.barrier)
    if cuda:
        t = heap.zeros((world,), torch.int64)
        for it in range(200):       # soak: jittered rounds (the reference runs 1000, test/nvidia/test_common_ops.py:54-92)
            if rng.random() < 0.5:
                torch.cuda._sleep(int(rng.random() * 2e6))
            t.local[rank] = it + 1
            CO.barrier_all_on_stream()
            got = torch.stack([t.peers[p][p].to(dev) for p in range(world)])
            CO.barrier_all_on_stream()
            assert (got == it + 1).all(), (it, got.tolist())
        check_status()
        res["barrier"] = "ok"

    # ---- all-gather, every mode, several sizes, byte-exact
    ag = {}
    for mode in (["pull", "push2d", "push_ordered", "push2d_ll"] if cuda else ["pull"]):
        for seg in ([512, 4096 + 8, 1 << 20] if cuda else [4096]):
            buf = heap.empty((world * seg,), torch.uint8)
            ctx = CO.create_fast_allgather_context(rank, 0, world, 1, max_buffer_size=world * seg, group=group, device=dev)
            for it in range(25 if (cuda and seg <= 8192) else 4):
                mine = torch.randint(0, 256, (seg,), dtype=torch.uint8, device=dev)
                heap.barrier()  # nobody is still reading the previous result
                buf.local.fill_(0xEE)
                buf.local[rank * seg:(rank + 1) * seg].copy_(mine)
                heap.barrier()  # every rank's buffer is prepared: a late fill must not wipe out a segment a peer already pushed
                if cuda and rng.random() < 0.5:
                    torch.cuda._sleep(int(rng.random() * 1e6))
                CO.fast_allgather(buf, ctx, mode=mode)
                exp = torch.empty(world * seg, dtype=torch.uint8, device=dev)
                dist.all_gather_into_tensor(exp, mine, group=group)
                assert torch.equal(buf.local, exp), (mode, seg, it)
            ag[f"{mode}/{seg}"] = "ok"
    if cuda:
        check_status()
    res["allgather"] = ag

    # ---- reduce-scatter: int32 exact, bf16 close
    for dtype in ([torch.int32, torch.bfloat16] if cuda else [torch.float32]):
        mpr, N = 96, 512
        M = world * mpr
        ctx = CO.create_reduce_scater_2d_ctx(M, N, rank, world, dtype=dtype, group=group, device=dev)
        for it in range(12 if cuda else 2):
            x = torch.randint(-100, 100, (M, N), device=dev).to(dtype)
            out = CO.reduce_scatter_2d_op(x, ctx)
            full = x.to(torch.float32)
            dist.all_reduce(full, group=group)
            ref = full[rank * mpr:(rank + 1) * mpr]
            assert torch.equal(out.to(torch.float32), ref) if dtype == torch.int32 else torch.allclose(out.float(), ref, atol=2.0, rtol=2e-2), (dtype, it)
    if cuda:
        check_status()
    res["reduce_scatter"] = "ok"

    ok = torch.ones(1, device=dev)
    dist.all_reduce(ok, group=group)
    res["ranks_ok"] = int(ok.item())
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    finalize_distributed()


if __name__ == "__main__":
    main()
