"""Per-op micro-benchmarks: device-timed, max over ranks, one JSON row per measurement.

    python -m triton_distributed_b200.bench_ops --op gemm --m 8192 --n 6144 --k 12288
    torchrun --nproc-per-node 8 -m triton_distributed_b200.bench_ops --op ag_gemm --m 8192 --n 49152 --k 12288

Rows carry {op, shape, world, us (max over ranks), tflops or gbps, roofline fraction}. The
roofline denominators are read from MEASURED_PEAKS.json at the repository root when present
(measured copy bandwidth and cuBLAS bf16 throughput of this machine), else the documented
fallback figures. The reference prints the same quantities per rank from its test scripts
(reference python/triton_dist/utils.py:186-198 `perf_func`, test_ag_gemm_intra_node.py perf mode).

`--iters 1 --warmup 0 --no-baseline` makes a run with exactly one launch of the op's kernel,
which is what a profiler capture wants.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d.get("hbm_gbs", 6650.0), "bf16_tflops": d.get("bf16_tflops", 1590.0),
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", 1400.0), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU on this pool


def timed_us(fn, iters: int, warmup: int, world: int, group=None) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier(group)
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["gemm", "ag_gemm", "gemm_rs"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=12288)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--cta-pair", type=int, default=-1)
    ap.add_argument("--no-baseline", action="store_true")
    args = ap.parse_args(argv)

    from .ops import gemm as G
    from .runtime import check_status, finalize_distributed, initialize_distributed

    world = int(os.environ.get("WORLD_SIZE", "1"))
    group = initialize_distributed(seed=0) if world > 1 or "RANK" in os.environ else None
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    G.CTA_PAIR = args.cta_pair
    pk = peaks()
    M, N, K = args.m, args.n, args.k
    row = {"op": args.op, "m": M, "n": N, "k": K, "world": world, "dtype": args.dtype, "peaks": pk["source"]}

    if args.op == "gemm":
        a = torch.randn(M, K, device=dev, dtype=dtype)
        b = (torch.randn(N, K, device=dev) * K ** -0.5).to(dtype)
        c = torch.empty(M, N, device=dev, dtype=dtype)
        us = timed_us(lambda: G.gemm_persistent(a, b, out=c), args.iters, args.warmup, 1)
        flops = 2.0 * M * N * K
        base = None if args.no_baseline else timed_us(lambda: torch.matmul(a, b.t(), out=c), args.iters, args.warmup, 1)
        link_us = 0.0
    elif args.op == "ag_gemm":
        mpr, npr = M // world, N // world
        a = torch.randn(mpr, K, device=dev, dtype=dtype)
        b = (torch.randn(npr, K, device=dev) * K ** -0.5).to(dtype)
        c = torch.empty(M, npr, device=dev, dtype=dtype)
        ctx = G.create_ag_gemm_intra_node_context(a, b, rank, world, max_M=M, group=group)
        us = timed_us(lambda: G.ag_gemm_intra_node(a, b, ctx, out=c), args.iters, args.warmup, world, group)
        flops = 2.0 * M * npr * K
        link_us = (world - 1) * mpr * K * 2 / (NVLINK_GBS * 1e3)
        base = None
        if not args.no_baseline:
            full = torch.empty(M, K, device=dev, dtype=dtype)

            def ref():
                if world > 1:
                    dist.all_gather_into_tensor(full, a, group=group)
                    torch.matmul(full, b.t(), out=c)
                else:
                    torch.matmul(a, b.t(), out=c)
            base = timed_us(ref, args.iters, args.warmup, world, group)
    else:
        mpr, kl = M // world, K // world
        a = torch.randn(M, kl, device=dev, dtype=dtype)
        b = (torch.randn(N, kl, device=dev) * K ** -0.5).to(dtype)
        o = torch.empty(mpr, N, device=dev, dtype=dtype)
        ctx = G.create_gemm_rs_context(M, N, rank, world, output_dtype=dtype, group=group, device=dev)
        us = timed_us(lambda: G.gemm_rs(a, b, ctx, out=o), args.iters, args.warmup, world, group)
        flops = 2.0 * M * N * kl
        link_us = (world - 1) * mpr * N * 2 / (NVLINK_GBS * 1e3)
        base = None
        if not args.no_baseline:
            full = torch.empty(M, N, device=dev, dtype=dtype)

            def ref():
                torch.matmul(a, b.t(), out=full)
                if world > 1:
                    dist.reduce_scatter_tensor(o, full, group=group)
            base = timed_us(ref, args.iters, args.warmup, world, group)
    check_status()
    compute_us = flops / (pk["bf16_tflops"] * 1e6)
    row.update({"us": round(us, 2), "tflops_per_gpu": round(flops / us / 1e6, 1),
                "roofline_us": round(max(compute_us, link_us), 2),
                "roofline_fraction": round(max(compute_us, link_us) / us, 3)})
    if base is not None:
        row.update({"torch_us": round(base, 2), "speedup_vs_torch": round(base / us, 3)})
    if rank == 0:
        print(json.dumps(row), flush=True)
    if dist.is_initialized():
        finalize_distributed()
    return 0


if __name__ == "__main__":
    sys.exit(main())
