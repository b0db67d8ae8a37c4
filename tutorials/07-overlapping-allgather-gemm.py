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
(reference tutorials/07-overlapping-allgather-gemm.py, kernels/nvidia/allgather_gemm.py)
"""
import torch
import torch.distributed as dist

from _common import dist_print, launch
from triton_distributed_b200.ops import gemm as G
from triton_distributed_b200.ops import gemm_fp8 as F8
from triton_distributed_b200.utils import perf_func


def run(group, rank, world, dev):
    cuda = dev.type == "cuda"
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


if __name__ == "__main__":
    launch(run)
