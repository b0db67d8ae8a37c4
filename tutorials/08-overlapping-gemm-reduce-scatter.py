"""Tutorial 08 — GEMM overlapped with ReduceScatter, in ONE kernel.

Row-parallel linear: rank r holds ``X_r [M, K/ws]`` and ``W_r [N, K/ws]``; the sum over ranks of
``X_r @ W_r^T`` leaves row-scattered. The fused kernel computes tiles in the order *peers' row blocks first,
own block last*; the epilogue of a tile stores it (TMA) straight into the owner's staging and raises the
tile's flag there; the tail of the same kernel waits for the world-1 senders of each of this rank's tiles and
adds them in fp32. The scatter of tile i overlaps the MMAs of tile i+1; only the last tile's transfer is
exposed. (reference tutorials/08-overlapping-gemm-reduce-scatter.py, kernels/nvidia/gemm_reduce_scatter.py)
"""
import torch
import torch.distributed as dist

from _common import dist_print, launch
from triton_distributed_b200.ops import gemm as G
from triton_distributed_b200.utils import perf_func


def run(group, rank, world, dev):
    cuda = dev.type == "cuda"
    M, N, K = (8192, 12288, 49152) if cuda else (64 * world, 128, 256 * world)
    dtype = torch.bfloat16 if cuda else torch.float32
    g = torch.Generator().manual_seed(rank)
    x = torch.randn(M, K // world, generator=g).to(dev, dtype)
    w = (torch.randn(N, K // world, generator=g) * K ** -0.5).to(dev, dtype)
    ctx = G.create_gemm_rs_context(M, N, rank, world, output_dtype=dtype, group=group, device=dev)
    y = G.gemm_rs(x, w, ctx)

    partial = x.float() @ w.float().t()
    ref = torch.empty(M // world, N, device=dev, dtype=torch.float32)
    if world > 1:
        dist.reduce_scatter_tensor(ref, partial, group=group) if cuda else ref.copy_(_cpu_rs(partial, rank, world, group))
    else:
        ref.copy_(partial)
    torch.testing.assert_close(y.float(), ref, atol=5e-2, rtol=3e-2)
    if cuda:
        full = torch.empty(M, N, device=dev, dtype=dtype)
        out = torch.empty(M // world, N, device=dev, dtype=dtype)

        def baseline():
            torch.matmul(x, w.t(), out=full)
            if world > 1:
                dist.reduce_scatter_tensor(out, full, group=group)
        _, ms = perf_func(lambda: G.gemm_rs(x, w, ctx), 10, 3)
        _, ms0 = perf_func(baseline, 10, 3)
        dist_print(f"fused GEMM-RS {ms:.3f} ms | cuBLAS + NCCL reduce-scatter {ms0:.3f} ms  (m{M} n{N} k{K}, tp{world})")
    dist_print("GEMM-RS ok")


def _cpu_rs(partial, rank, world, group):
    total = partial.clone()
    dist.all_reduce(total, group=group)
    per = total.shape[0] // world
    return total[rank * per:(rank + 1) * per]


if __name__ == "__main__":
    launch(run)
