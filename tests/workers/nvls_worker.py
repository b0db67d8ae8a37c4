"""Multi-rank check of the NVLS (multimem) collectives against NCCL / gloo oracles.

On CUDA the heap is created with TDIST_NVLS=1, so every symmetric tensor has a multicast alias. Whatever
happens, every rank reaches the final barrier and closes its heap (unbinding its memory from the multicast
object) before it exits.
"""
import json
import traceback

import torch
import torch.distributed as dist

from triton_distributed_b200.ops import collectives as CO
from triton_distributed_b200.ops import nvls as NV
from triton_distributed_b200.runtime import check_status, finalize_distributed, initialize_distributed, symm_heap


def body(group, rank, world, dev, cuda, res):
    heap = symm_heap(group)
    ctx = NV.create_nvls_context(rank, world, heap=heap, group=group, device=dev)
    probe = heap.empty((world * 64,), torch.float32)
    res["multicast"] = bool(NV.nvls_available(probe)) if cuda else False
    if cuda and not res["multicast"]:
        return
    sizes = [world * 1024, world * 250 * 264, world * (1 << 20)] if cuda else [world * 256]
    for dtype in ([torch.bfloat16, torch.float32, torch.float16] if cuda else [torch.float32]):
        for n in sizes:
            seg = n // world
            buf = heap.empty((n,), dtype)
            for it in range(3 if cuda else 1):
                gen = torch.Generator(device="cpu").manual_seed(1000 * it + n % 997)
                full = [torch.randn(n, generator=gen) for _ in range(world)]   # every rank's whole copy
                mine = full[rank].to(dev, dtype)
                # ---- all-gather
                buf.local.fill_(float("nan"))
                buf.local[rank * seg:(rank + 1) * seg].copy_(mine[rank * seg:(rank + 1) * seg])
                heap.barrier()
                NV.nvls_allgather(buf, ctx)
                if cuda:
                    check_status()
                want = torch.cat([full[r][r * seg:(r + 1) * seg] for r in range(world)]).to(dev, dtype)
                assert torch.equal(buf.local, want), f"allgather {dtype} n={n} it={it}"
                heap.barrier()
                # ---- reduce-scatter
                buf.local.copy_(mine)
                heap.barrier()
                out = NV.nvls_reduce_scatter(buf, ctx)
                if cuda:
                    check_status()
                ref = sum(f.to(dev, dtype).float() for f in full)
                tol = dict(atol=2e-2, rtol=2e-2) if dtype != torch.float32 else dict(atol=1e-4, rtol=1e-5)
                torch.testing.assert_close(out.float(), ref[rank * seg:(rank + 1) * seg], **tol)
                heap.barrier()
                # ---- all-reduce (in place)
                buf.local.copy_(mine)
                heap.barrier()
                NV.nvls_allreduce(buf, ctx)
                if cuda:
                    check_status()
                torch.testing.assert_close(buf.local.float(), ref, **tol)
                heap.barrier()
    # fast_allgather's multimem mode routes to the NVLS kernel
    if cuda:
        ag = CO.create_fast_allgather_context(rank, num_ranks=world, group=group, device=dev)
        buf = heap.empty((world * 4096,), torch.int32)
        buf.local.fill_(-1)
        buf.local[rank * 4096:(rank + 1) * 4096] = rank + 7
        heap.barrier()
        CO.fast_allgather(buf, ag, mode="push2d_ll_multimem")
        check_status()
        want = torch.arange(world, device=dev, dtype=torch.int32).repeat_interleave(4096) + 7
        assert torch.equal(buf.local, want)
        res["fast_allgather_used_nvls"] = bool(ag.nvls is not None and ag.nvls.epoch > 0)
        heap.barrier()
    # the sequence-parallel decode exchanges its partial results as LL packets stored once through the multicast alias
    if cuda:
        import math

        from triton_distributed_b200.ops import flash_decode as FD
        B, Hq, Hkv, D, page = 4, 32, 8, 128, 16
        sctx = FD.create_sp_decode_context(rank, world, B, Hq, D, group=group, device=dev)
        res["sp_decode_multicast"] = bool(sctx.gather.mc is not None and FD.SP_DECODE_NVLS)
        for it in range(6):
            gen = torch.Generator().manual_seed(55 + it)  # identical on every rank
            q = torch.randn(B, Hq, D, generator=gen).to(dev, torch.bfloat16)
            glens = torch.randint(1, 600, (world, B), generator=gen, dtype=torch.int32).to(dev)
            max_blocks = (int(glens[rank].max()) + page - 1) // page
            k = torch.randn(B * max_blocks, page, Hkv, D, device=dev).to(torch.bfloat16)
            v = torch.randn(B * max_blocks, page, Hkv, D, device=dev).to(torch.bfloat16)
            table = torch.randperm(B * max_blocks, device=dev).view(B, max_blocks).to(torch.int32)
            out = FD.sp_gqa_fwd_batch_decode(sctx, q, k, v, glens, table)
            check_status()
            o, l = FD.ref_paged_attn(q, k, v, glens[rank], table, 1.0 / math.sqrt(D), return_lse=True)
            mine = torch.cat([o, l.unsqueeze(-1)], -1).contiguous()
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine, group=group)
            ref = FD.ref_lse_merge(torch.stack(parts))
            torch.testing.assert_close(out.float(), ref, atol=5e-2, rtol=5e-2)
    res["checked"] = True


def main():
    group = initialize_distributed(seed=0)
    rank, world = dist.get_rank(), dist.get_world_size()
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    res = {"world": world, "device": dev.type, "checked": False}
    good = 1
    try:
        body(group, rank, world, dev, cuda, res)
    except Exception:  # noqa: BLE001 - every rank must still reach the barrier below and close its heap
        good = 0
        res["error"] = traceback.format_exc()[-1500:]
        print(res["error"], flush=True)
    ok = torch.tensor([float(good)], device=dev)
    dist.all_reduce(ok, group=group)
    res["ranks_ok"] = int(ok.item())
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    finalize_distributed()


if __name__ == "__main__":
    main()
