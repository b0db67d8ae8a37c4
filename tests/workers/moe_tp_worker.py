"""Multi-rank check of the tensor-parallel MoE ops: AG + GroupGEMM and GroupGEMM + top-k reduce + reduce-scatter, in
every launch mode, against an fp32 restatement over the all-gathered inputs (NCCL / gloo as the oracle for the
collectives). Fresh tokens every iteration on one context, as in serving; some ranks start late so that the grouped
GEMM really meets segments that have not arrived. Follows the reference's test_ag_moe.py / test_moe_reduce_rs.py
(test/nvidia/test_ag_moe.py:120-210, test/nvidia/test_moe_reduce_rs.py:150-260)."""
import json
import random

import torch
import torch.distributed as dist

from triton_distributed_b200.ops import moe_tp as MT
from triton_distributed_b200.runtime import check_status, finalize_distributed, initialize_distributed


def main():
    group = initialize_distributed(seed=0)
    rank, world = dist.get_rank(), dist.get_world_size()
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    rng = random.Random(rank)
    res = {"world": world, "device": dev.type}
    shapes = [(96, 512, 256, 8, 2), (200, 1024, 264, 6, 3)] if cuda else [(16, 64, 32, 4, 2)]   # tokens/rank, K, N/rank, E, topk
    modes = ["fused", "staged", "cp_async"] if cuda else ["staged"]
    ag_err = rs_err = 0.0
    for (tpr, K, n_per, E, topk) in shapes:
        M = tpr * world
        gen = torch.Generator().manual_seed(7)
        ids = torch.randint(0, E, (M, topk), generator=gen, dtype=torch.int32).to(dev)
        wts = torch.rand(M, topk, generator=gen).to(dev)
        w1 = (torch.randn(E, K, world * n_per, generator=gen) * K ** -0.5)[:, :, rank * n_per:(rank + 1) * n_per].to(dev, dtype).contiguous()
        # second op: rows are (token, k) pairs with n_per features each, weights [E, n_per, K] per rank
        w2 = (torch.randn(E, world * n_per, K, generator=gen) * (world * n_per) ** -0.5)[:, rank * n_per:(rank + 1) * n_per].to(dev, dtype).contiguous()
        for mode in modes:
            MT.AG_GROUP_GEMM_MODE = mode
            ctx = MT.create_ag_group_gemm_intra_node_context(group, torch.empty(tpr, K, dtype=dtype, device=dev), w1, ids, E,
                                                             max_M=M, rank=rank, num_ranks=world)
            rctx = MT.create_moe_rs_context(group, rank, world, world, M, K, E, topk, dtype, dtype, dev, full_topk_ids=ids,
                                            full_topk_weight=wts)
            for it in range(6 if cuda else 1):
                x_full = torch.randn(M, K, generator=gen)
                x = x_full[rank * tpr:(rank + 1) * tpr].to(dev, dtype).contiguous()
                if cuda and rng.random() < 0.5:
                    torch.cuda._sleep(int(rng.random() * 2e6))     # a late rank: its segment is missing when the others start
                h = MT.ag_group_gemm_intra_node(x, w1, ctx)
                if cuda:
                    check_status()
                xf = x_full.to(dtype).float().to(dev)
                flat = ids.reshape(-1).long()
                want = torch.empty(M * topk, n_per, device=dev)
                rows = xf[torch.arange(M * topk, device=dev) // topk]
                for e in range(E):
                    m = flat == e
                    want[m] = rows[m] @ w1[e].float()
                torch.testing.assert_close(h.float(), want, atol=3e-2 if cuda else 1e-4, rtol=3e-2 if cuda else 1e-4)
                ag_err = max(ag_err, (h.float() - want).abs().max().item())

                out = MT.moe_reduce_rs(rank, world, world, h, w2, rctx)
                if cuda:
                    check_status()
                y = torch.empty(M * topk, K, device=dev)
                hf = h.float()
                for e in range(E):
                    m = flat == e
                    y[m] = hf[m] @ w2[e].float()
                part = (y.view(M, topk, K) * wts.view(M, topk, 1)).sum(1)
                dist.all_reduce(part, group=group)
                ref = part[rank * tpr:(rank + 1) * tpr]
                torch.testing.assert_close(out.float(), ref, atol=6e-2 if cuda else 1e-4, rtol=5e-2 if cuda else 1e-4)
                rs_err = max(rs_err, (out.float() - ref).abs().max().item())
    res["ag_group_gemm_max_err"] = ag_err
    res["moe_reduce_rs_max_err"] = rs_err
    res["modes"] = modes
    ok = torch.ones(1, device=dev)
    dist.all_reduce(ok, group=group)
    res["ranks_ok"] = int(ok.item())
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    finalize_distributed()


if __name__ == "__main__":
    main()
