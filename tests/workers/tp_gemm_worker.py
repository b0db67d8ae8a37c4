"""Multi-rank check of the symmetric heap and the fused AG-GEMM / GEMM-RS ops.

Runs under torchrun on CUDA (NCCL oracle: all_gather_into_tensor + matmul, matmul +
reduce_scatter_tensor) or on CPU (gloo plumbing config: fp32, seed 0, rtol 1e-5).
Follows the reference's test_ag_gemm_intra_node.py:129-149 and test_gemm_rs.py:43-115:
fresh random inputs every iteration, non-tile-aligned M, stale-workspace poisoning.
"""
import json
import sys

import torch
import torch.distributed as dist

from triton_distributed_b200.ops import gemm as G
from triton_distributed_b200.ops import gemm_fp8 as F8
from triton_distributed_b200.runtime import check_status, finalize_distributed, initialize_distributed, symm_heap


ITERS = 20   # fresh-data iterations per small shape (one context reused, as in serving)


def main():
    group = initialize_distributed(seed=0)
    rank, world = dist.get_rank(), dist.get_world_size()
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    res = {"world": world, "device": dev.type}

    if cuda:
        heap = symm_heap(group)
        t = heap.zeros((world, 16), torch.int32)
        t.local[rank].fill_(rank + 1)
        heap.barrier()
        seen = [int(t.peers[p].to(dev)[p, 0].item()) for p in range(world)]
        res["heap_backend"] = heap._segments[0].cleanup is not None and ("vmm" if hasattr(heap._segments[0], "base_va") else "ipc")
        assert seen == [p + 1 for p in range(world)], seen
        heap.barrier()

    # ---------------- AG-GEMM ----------------
    # on GPUs: tile-aligned, ragged (8-column partial tile, rows no multiple of 128), and two K >= 4096 problems that the
    # launcher runs with the wide (256 x 512) pair tiling, one of them with a 200-column partial tile; the last one has
    # 44 wide items per segment (21 tiles per row: an odd one out) for ~70 CTA pairs, so its first round is split in halves
    shapes = [(128, 256, 256), (999, 264, 520)] if cuda else [(128, 256, 256)]
    if cuda:
        shapes += [(1024, 1024, 2048), (520, 1224, 4096), (256, 2048, 4160), (1000, 5128, 4096)]
    ag_err = 0.0
    for (mpr, n_per, K) in shapes:
        gen = torch.Generator(device="cpu").manual_seed(0)
        ctx = None
        for it in range((ITERS if mpr * K <= 1 << 21 else 3) if cuda else 1):
            A_full = torch.randn(world * mpr, K, generator=gen)
            W_full = torch.randn(world * n_per, K, generator=gen) * (0.02 if not cuda else K ** -0.5)
            a = A_full[rank * mpr:(rank + 1) * mpr].to(dev, dtype).contiguous()
            w = W_full[rank * n_per:(rank + 1) * n_per].to(dev, dtype).contiguous()
            if ctx is None:
                ctx = G.create_ag_gemm_intra_node_context(a, w, rank, world, max_M=world * mpr, group=group,
                                                          for_correctness=(it == 0))
            if cuda and ctx.workspace is not None:
                ctx.workspace.local.fill_(float("nan"))  # stale data must never be consumed
                symm_heap().barrier()
            c = G.ag_gemm_intra_node(a, w, ctx)
            if cuda:
                check_status()
            gathered = torch.empty(world * mpr, K, device=dev, dtype=dtype)
            dist.all_gather_into_tensor(gathered, a, group=group)
            ref = gathered.float() @ w.float().t()
            if cuda:
                torch.testing.assert_close(c.float(), ref, atol=2e-2, rtol=2e-2)
            else:
                torch.testing.assert_close(c, ref, rtol=1e-5, atol=1e-5)
                torch.testing.assert_close(c, A_full @ w.t(), rtol=1e-5, atol=1e-5)
            ag_err = max(ag_err, (c.float() - ref).abs().max().item())
            if cuda:
                symm_heap().barrier()
    res["ag_max_err"] = ag_err
    res["ag_multicast_pusher"] = bool(cuda and ctx is not None and ctx.workspace is not None and ctx.workspace.mc is not None and (G.AG_NVLS == 2 or world >= 4))

    # ---------------- GEMM-RS ----------------
    shapes = [(128, 256, 128), (250, 520, 264), (1024, 2048, 1024), (300, 1224, 4096)] if cuda else [(128, 256, 128)]
    rs_err = 0.0
    for (mpr, N, k_loc) in shapes:
        gen = torch.Generator(device="cpu").manual_seed(0)
        M = world * mpr
        ctx = G.create_gemm_rs_context(M, N, rank, world, output_dtype=dtype, group=group, device=dev)
        for it in range((ITERS if M * k_loc <= 1 << 21 else 3) if cuda else 1):
            X_full = torch.randn(M, world * k_loc, generator=gen)
            V_full = torch.randn(N, world * k_loc, generator=gen) * (0.02 if not cuda else (world * k_loc) ** -0.5)
            x = X_full[:, rank * k_loc:(rank + 1) * k_loc].to(dev, dtype).contiguous()
            v = V_full[:, rank * k_loc:(rank + 1) * k_loc].to(dev, dtype).contiguous()
            out = G.gemm_rs(x, v, ctx)
            if cuda:
                check_status()
            partial = x.float() @ v.float().t()
            if cuda:
                ref = torch.empty(mpr, N, device=dev, dtype=torch.float32)
                dist.reduce_scatter_tensor(ref, partial, group=group)
                torch.testing.assert_close(out.float(), ref, atol=3e-2, rtol=3e-2)
            else:
                ref = (X_full @ V_full.t())[rank * mpr:(rank + 1) * mpr]
                torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
            rs_err = max(rs_err, (out.float() - ref).abs().max().item())
    res["rs_max_err"] = rs_err

    # ---------------- block-scaled fp8 AG-GEMM ----------------
    # oracle: all_gather of rows and scales (NCCL / gloo), then the fp32 matmul of the dequantised operands
    f8_err = 0.0
    for (mpr, n_per, K) in ([(128, 256, 256), (250, 264, 384), (1024, 1024, 2048)] if cuda else [(64, 128, 256)]):
        gen = torch.Generator(device="cpu").manual_seed(1)
        ctx = F8.create_ag_gemm_fp8_context(world * mpr, K, rank, world, device=dev, group=group)
        for it in range(3 if cuda else 1):
            X = torch.randn(world * mpr, K, generator=gen)
            Wt = torch.randn(world * n_per, K, generator=gen) * K ** -0.5
            a, sa = F8.quantize_fp8_rowwise(X[rank * mpr:(rank + 1) * mpr].to(dev))
            b, sb = F8.quantize_fp8_blockwise(Wt[rank * n_per:(rank + 1) * n_per].to(dev))
            if cuda and ctx.workspace is not None:
                ctx.workspace.local.fill_(0x7F)          # stale rows (e4m3 NaN) must never be consumed
                ctx.scale_ws.local.fill_(float("nan"))
                symm_heap().barrier()
            c = F8.ag_gemm_fp8(a, sa, b, sb, ctx)
            if cuda:
                check_status()
            rows = torch.empty(world * mpr, K, device=dev, dtype=torch.uint8)
            scales = torch.empty(world * mpr, K // 128, device=dev, dtype=torch.float32)
            dist.all_gather_into_tensor(rows, a.view(torch.uint8).contiguous(), group=group)
            dist.all_gather_into_tensor(scales, sa.contiguous(), group=group)
            ref = F8.dequantize_fp8(rows.view(F8.FP8), scales, 1) @ F8.dequantize_fp8(b, sb, 128).t()
            assert torch.isfinite(c.float()).all()
            torch.testing.assert_close(c.float(), ref, atol=5e-3 * ref.abs().max().item(), rtol=1e-2)
            f8_err = max(f8_err, (c.float() - ref).abs().max().item())
            if cuda:
                symm_heap().barrier()
    res["fp8_ag_max_err"] = f8_err

    ok = torch.ones(1, device=dev)
    dist.all_reduce(ok, group=group)
    res["ranks_ok"] = int(ok.item())
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    finalize_distributed()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        # leave in an orderly way: the heap is closed (memory unbound from any multicast object) before exit
        import traceback
        traceback.print_exc()
        try:
            finalize_distributed()
        except Exception:  # noqa: BLE001
            pass
        sys.exit(1)
