"""Tutorial 07 — AllGather overlapped with GEMM, in ONE kernel.

Column-parallel linear with sequence-parallel input: rank r holds ``A_r [M/ws, K]`` and ``W_r [N/ws, K]`` and
needs ``allgather(A) @ W_r^T``. The fused kernel is a persistent grid in which

* a few *pusher* CTAs stream this rank's rows into every peer's gather workspace with bulk (TMA) copies and
  raise one flag per 128-row block on the destination;
* the other CTAs are a tcgen05 GEMM (TMA -> shared memory -> ``tcgen05.mma`` -> TMEM -> epilogue). Tiles are
  visited own-segment-first, then in the order the peers' blocks arrive; the TMA producer of a tile waits on
  the flag of exactly the block it is about to load.

No side stream, no copy engine, no host-side signalling; flags carry the call number, the workspace is
double-buffered by call parity, so calls need no barrier between them.

The script first runs ``tutorials/kernels/overlap_gemm.cu``: the same kernel structure (pusher CTAs, per-block flags,
consumers that start on their own rows and wait block by block) in ~60 lines with a plain dot product where the
production kernel has its tcgen05 pipeline. Read that file first; the comments marked PRODUCTION say what
``csrc/kernels/gemm_sm100.cu`` adds. Then the production op on the full-size problem, against NCCL + cuBLAS.
(reference tutorials/07-overlapping-allgather-gemm.py, kernels/nvidia/allgather_gemm.py)
"""
import torch
import torch.distributed as dist

from _common import dist_print, launch
from triton_distributed_b200.ops import gemm as G
from triton_distributed_b200.ops import gemm_fp8 as F8
from triton_distributed_b200.utils import perf_func


def skeleton(group, rank, world, dev):
    """The teaching kernel: fp32, small, two calls on the same workspace (flags carry the call number)."""
    from triton_distributed_b200.runtime import check_status, default_timeout_ns, global_status, symm_heap
    lib = _overlap_lib()
    heap = symm_heap(group)
    mpr, N, K = 72, 200, 96                                    # ragged on purpose: 16-row blocks and 16-wide tiles
    ws = heap.empty((world, mpr, K), torch.float32)            # every rank's gather workspace
    flags = heap.zeros((world * ((mpr + 15) // 16),), torch.int32)
    b = torch.randn(N, K, device=dev)
    for call in (1, 2):
        a = torch.randn(mpr, K, device=dev)
        ws.local.fill_(float("nan"))                           # stale rows must never be consumed
        heap.barrier()                                         # demo only (the production op double-buffers instead)
        out = torch.empty(world * mpr, N, device=dev)
        rc = lib.tutorial_overlap_launch(0, ws.ptr_array(), flags.ptr_array(), a.data_ptr(), b.data_ptr(), out.data_ptr(), mpr, N, K,
                                         rank, world, 4, call, global_status().device_ptr, default_timeout_ns(),
                                         torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        check_status()
        full = torch.empty(world * mpr, K, device=dev)
        if world > 1:
            dist.all_gather_into_tensor(full, a, group=group)
        else:
            full.copy_(a)
        torch.testing.assert_close(out, full @ b.t(), atol=1e-3, rtol=1e-3)
        heap.barrier()
    dist_print("AG-GEMM skeleton (user kernel: pushers + per-block waits) ok")


def run(group, rank, world, dev):
    cuda = dev.type == "cuda"
    if cuda:
        skeleton(group, rank, world, dev)
    M, N, K = (8192, 49152, 12288) if cuda else (64 * world, 128 * world, 256)
    dtype = torch.bfloat16 if cuda else torch.float32
    g = torch.Generator().manual_seed(rank)
    a = torch.randn(M // world, K, generator=g).to(dev, dtype)
    w = (torch.randn(N // world, K, generator=g) * K ** -0.5).to(dev, dtype)
    ctx = G.create_ag_gemm_intra_node_context(a, w, rank, world, max_M=M, group=group)
    c = G.ag_gemm_intra_node(a, w, ctx)

    full = torch.empty(M, K, device=dev, dtype=dtype)
    if world > 1:
        dist.all_gather_into_tensor(full, a, group=group)
    else:
        full.copy_(a)
    torch.testing.assert_close(c.float(), full.float() @ w.float().t(), atol=3e-2, rtol=3e-2)

    # the fp8 flavour: e4m3 rows with 1x128 scales, weights with 128x128 scales; rows AND scales are gathered in-kernel
    a8, sa = F8.quantize_fp8_rowwise(a)
    w8, sw = F8.quantize_fp8_blockwise(w)
    ctx8 = F8.create_ag_gemm_fp8_context(M, K, rank, world, device=dev, group=group)
    c8 = F8.ag_gemm_fp8(a8, sa, w8, sw, ctx8)
    assert c8.shape == c.shape and torch.isfinite(c8.float()).all()

    if cuda:
        def baseline():
            if world > 1:
                dist.all_gather_into_tensor(full, a, group=group)
            torch.matmul(full, w.t())
        _, ms = perf_func(lambda: G.ag_gemm_intra_node(a, w, ctx), 10, 3)
        _, ms8 = perf_func(lambda: F8.ag_gemm_fp8(a8, sa, w8, sw, ctx8), 10, 3)
        _, ms0 = perf_func(baseline, 10, 3)
        dist_print(f"fused AG-GEMM {ms:.3f} ms | fp8 {ms8:.3f} ms | NCCL all-gather + cuBLAS {ms0:.3f} ms  (m{M} n{N} k{K}, tp{world})")
    dist_print("AG-GEMM ok")


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
