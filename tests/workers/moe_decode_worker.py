"""Multi-rank check of the MoE all-to-all (generic + fused fp8 dispatch / weighted combine) and of
the sequence-parallel flash decode. Oracles are torch restatements evaluated on gathered inputs
(the reference compares against NCCL all_to_all_single and a global paged attention:
test_all_to_all.py:184-241,350-367; test_sp_decode_attn.py:81-131)."""
import json
import math

import torch
import torch.distributed as dist

from triton_distributed_b200.ops import all_to_all as A
from triton_distributed_b200.ops import flash_decode as FD
from triton_distributed_b200.ops import moe_utils as MU
from triton_distributed_b200.runtime import check_status, finalize_distributed, initialize_distributed


def gather_list(t, group, world):
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t.contiguous(), group=group)
    return out


def main():
    group = initialize_distributed(seed=0)
    rank, world = dist.get_rank(), dist.get_world_size()
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    res = {"world": world, "device": dev.type}
    torch.manual_seed(1234 + rank)

    # ---------------- generic fast_all_to_all: dispatch, then combine back, like the reference test
    T, H, K = (128, 1024, 4) if cuda else (16, 128, 2)
    E = 8 * world
    epr = E // world
    ctx = A.create_all_to_all_context(T * K, H, rank, E, world, epr, dtype=torch.bfloat16 if cuda else torch.float32,
                                      group=group, device=dev)
    for it in range(3):
        x = torch.randn(T, H, device=dev).to(ctx.dtype)
        ids = torch.randint(0, E, (T, K), dtype=torch.int32, device=dev)
        rt = MU.route(ids, E)
        send = x[rt.sorted_token.long()].contiguous()
        splits, recv, _ = A.fast_all_to_all(ctx, send, rt.cumsum, None)
        data, _ = A.all_to_all_post_process(ctx, splits, recv, None)
        # oracle: what every source sends to me
        all_send = gather_list(send, group, world)
        all_cum = gather_list(rt.cumsum, group, world)
        want = torch.cat([all_send[s][int(all_cum[s][rank * epr]): int(all_cum[s][(rank + 1) * epr])] for s in range(world)])
        assert torch.equal(data, want), ("dispatch", it)
        # combine with the received splits: every row returns to its sorted position
        cums = torch.zeros(E + 1, dtype=torch.int32, device=dev)
        cums[1:] = torch.cumsum(splits.reshape(-1), 0)
        _s2, back, _ = A.fast_all_to_all(ctx, data.contiguous(), cums, None)
        per_rank = [int(rt.cumsum[(d + 1) * epr]) - int(rt.cumsum[d * epr]) for d in range(world)]
        got = torch.cat([back[d * T * K: d * T * K + per_rank[d]] for d in range(world)])
        assert torch.equal(got, send), ("combine", it)
        if cuda:
            check_status()
    res["fast_all_to_all"] = "ok"

    # ---------------- fused fp8 dispatch + weighted combine with identity experts
    T, H, K = (128, 7168, 8) if cuda else (8, 256, 2)
    E = 32 * world if cuda else 4 * world
    mctx = A.create_moe_dispatch_context(T, H, K, E, rank, world, group=group, device=dev)
    err = 0.0
    for it in range(3):
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        ids, w = MU.topk_softmax(torch.randn(T, E, device=dev), K)
        rx, rs, splits = A.moe_dispatch(mctx, x, ids, w)
        y = A.dequant_fp8(rx, rs)
        out = A.moe_combine(mctx, y, splits)
        if cuda:
            check_status()
        q, sc = A.quant_fp8_reference(x)
        deq = (q.float().view(T, H // 128, 128) * sc.unsqueeze(-1)).view(T, H).to(torch.bfloat16).float()
        ref = deq * w.sum(-1, keepdim=True)
        err = max(err, (out.float() - ref).abs().max().item())
        assert torch.allclose(out.float(), ref, atol=3e-2, rtol=3e-2), ("fused", it, err)
    res["fused_moe_err"] = err

    # ---------------- expert-parallel layer: dispatched rows against all_to_all_single, exactly
    # (the reference's check: test/nvidia/test_ep_a2a.py:206-264)
    from triton_distributed_b200.models import EPAll2AllLayer
    T, H, K = (96, 512, 4) if cuda else (8, 64, 2)
    E = 8 * world
    epr = E // world
    layer = EPAll2AllLayer(group, T, H, K, rank, E, world, world, device=dev)
    for it in range(3):
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        ids = torch.randint(0, E, (T, K), dtype=torch.int32, device=dev)
        rows = layer.dispatch(x, ids)
        if cuda:
            check_status()
        n = int(layer.num_recv)
        # oracle: expert-sorted rows, exchanged with the collective, then regrouped from (source, expert) to (expert, source)
        rt = MU.route(ids, E)
        send = x[rt.sorted_token.long()].contiguous()
        counts = torch.stack(gather_list(rt.splits, group, world)).long()                 # [source, expert]
        mine = counts[:, rank * epr:(rank + 1) * epr]                                    # [source, local expert]
        in_splits = [int(v) for v in counts[rank].view(world, epr).sum(1)]
        out_splits = [int(v) for v in mine.sum(1)]
        got = torch.empty((sum(out_splits), H), dtype=send.dtype, device=dev)
        if cuda:
            dist.all_to_all_single(got, send, out_splits, in_splits, group=group)
        else:   # gloo has no all_to_all_single on every build: gather everything and cut
            every = gather_list(torch.cat([send, send.new_zeros((T * K - send.shape[0], H))]), group, world)
            every_cum = gather_list(rt.cumsum, group, world)
            got = torch.cat([every[s][int(every_cum[s][rank * epr]): int(every_cum[s][(rank + 1) * epr])] for s in range(world)])
        per_src = torch.split(got, out_splits)
        want = []
        for le in range(epr):
            for s_ in range(world):
                lo = int(mine[s_, :le].sum())
                want.append(per_src[s_][lo: lo + int(mine[s_, le])])
        want = torch.cat(want)
        assert n == want.shape[0], ("ep rows", it, n, want.shape[0])
        assert torch.equal(rows[:n], want), ("ep dispatch", it)
        out = layer.combine(rows)
        if cuda:
            check_status()
        assert torch.allclose(out.float(), x.float() * K, atol=2e-2, rtol=2e-2), ("ep combine", it)
    res["ep_layer"] = "ok"

    # ---------------- sequence-parallel decode
    B, Hq, Hkv, D, page = (4, 32, 8, 128, 16) if cuda else (2, 8, 2, 64, 4)
    dtype = torch.bfloat16 if cuda else torch.float32
    sctx = FD.create_sp_decode_context(rank, world, B, Hq, D, group=group, device=dev)
    derr = 0.0
    for it in range(4):
        gen = torch.Generator().manual_seed(77 + it)  # identical on every rank
        q = torch.randn(B, Hq, D, generator=gen).to(dev, dtype)
        glens = torch.randint(0, 700 if cuda else 20, (world, B), generator=gen, dtype=torch.int32)
        glens[0, 0] = 9
        if it == 2 and world > 1:
            glens[1] = 0
        glens = glens.to(dev)
        n_mine = [max(1, int(v)) for v in glens[rank]]
        max_blocks = (max(n_mine) + page - 1) // page
        k = torch.randn(B * max_blocks, page, Hkv, D, device=dev).to(dtype)
        v = torch.randn(B * max_blocks, page, Hkv, D, device=dev).to(dtype)
        table = torch.randperm(B * max_blocks, device=dev).view(B, max_blocks).to(torch.int32)
        out = FD.sp_gqa_fwd_batch_decode(sctx, q, k, v, glens, table)
        if cuda:
            check_status()
        o, l = FD.ref_paged_attn(q, k, v, glens[rank], table, 1.0 / math.sqrt(D), return_lse=True)
        parts = torch.stack(gather_list(torch.cat([o, l.unsqueeze(-1)], -1), group, world))
        ref = FD.ref_lse_merge(parts)
        derr = max(derr, (out.float() - ref).abs().max().item())
        assert torch.allclose(out.float(), ref, atol=5e-2, rtol=5e-2), ("sp_decode", it, derr)
    res["sp_decode_err"] = derr

    ok = torch.ones(1, device=dev)
    dist.all_reduce(ok, group=group)
    res["ranks_ok"] = int(ok.item())
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    finalize_distributed()


if __name__ == "__main__":
    main()
