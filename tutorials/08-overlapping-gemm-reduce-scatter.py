"""Tutorial 08 — GEMM overlapped with ReduceScatter, in ONE kernel.

Row-parallel linear: rank r holds ``X_r [M, K/ws]`` and ``W_r [N, K/ws]``; the sum over ranks of
``X_r @ W_r^T`` leaves row-scattered. The fused kernel computes tiles in the order *peers' row blocks first,
own block last*; the epilogue of a tile stores it (TMA) straight into the owner's staging and raises the
tile's flag there; the epilogue of one of this rank's OWN tiles instead waits for the world-1 senders of that tile,
adds their partials to the accumulator in fp32 and writes the finished rows. The scatter of tile i overlaps the MMAs
of tile i+1; only the last tile's transfer is exposed, and there is no reduce pass after the GEMM.

The script first runs the GEMM-RS half of ``tutorials/kernels/overlap_gemm.cu``: the same structure (tiles in
"remote owners first" order, epilogue stores into the owner's staging, one flag per (tile, source), reduce tail) with a
plain dot product in place of the tcgen05 pipeline; its comments marked PRODUCTION say what the real kernel adds.
(reference tutorials/08-overlapping-gemm-reduce-scatter.py, kernels/nvidia/gemm_reduce_scatter.py)
"""
import torch
import torch.distributed as dist

from _common import dist_print, launch
from triton_distributed_b200.ops import gemm as G
from triton_distributed_b200.utils import perf_func


def skeleton(group, rank, world, dev):
    from triton_distributed_b200.runtime import check_status, default_timeout_ns, global_status, symm_heap
    lib = _overlap_lib()
    heap = symm_heap(group)
    mpr, N, Kl = 40, 72, 64
    stage = heap.empty((world, mpr, N), torch.float32)         # staging: slot s = partial rows from source s
    tiles = ((mpr + 15) // 16) * ((N + 15) // 16)
    flags = heap.zeros((tiles * world,), torch.int32)
    for call in (1, 2):
        x = torch.randn(world * mpr, Kl, device=dev)
        w = torch.randn(N, Kl, device=dev)
        stage.local.fill_(float("nan"))
        heap.barrier()                                         # demo only (the production op double-buffers instead)
        out = torch.empty(mpr, N, device=dev)
        rc = lib.tutorial_overlap_launch(1, stage.ptr_array(), flags.ptr_array(), x.data_ptr(), w.data_ptr(), out.data_ptr(), mpr, N,
                                         Kl, rank, world, 0, call, global_status().device_ptr, default_timeout_ns(),
                                         torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        check_status()
        partial = x @ w.t()
        ref = torch.empty(mpr, N, device=dev)
        if world > 1:
            dist.reduce_scatter_tensor(ref, partial, group=group)
        else:
            ref.copy_(partial)
        torch.testing.assert_close(out, ref, atol=1e-3, rtol=1e-3)
        heap.barrier()
    dist_print("GEMM-RS skeleton (user kernel: epilogue scatter + per-tile flags + reduce tail) ok")


def run(group, rank, world, dev):
    cuda = dev.type == "cuda"
    if cuda:
        skeleton(group, rank, world, dev)
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


def _overlap_lib():
    import ctypes as C
    import os

    from triton_distributed_b200.utils.user_kernels import load_user_library
    lib = load_user_library(os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernels", "overlap_gemm.cu"))
    lib.tutorial_overlap_launch.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                            C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint, C.c_void_p, C.c_ulonglong, C.c_void_p]
    return lib


if __name__ == "__main__":
    launch(run)
