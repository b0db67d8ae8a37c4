"""Per-op micro-benchmarks: device-timed, max over ranks, one JSON row per measurement.

    python -m triton_distributed_b200.bench_ops --op gemm --m 8192 --n 6144 --k 12288
    torchrun --nproc-per-node 8 -m triton_distributed_b200.bench_ops --op ag_gemm --shape 8192x49152x12288

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


PRESLEEP_CYCLES = 0  # set by --presleep-ms: a spin kernel queued ahead of the timed launches


def timed_us(fn, iters: int, warmup: int, world: int, group=None) -> float:
    """Device time per call over `iters` back-to-back calls, max over ranks. With a pre-sleep the
    host enqueues all timed launches while the GPU is still spinning, so the figure excludes host
    launch overhead (the reference does the same: test_fast_allgather.py `torch.cuda._sleep(1e9)`)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier(group)
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if PRESLEEP_CYCLES > 0:
        torch.cuda._sleep(PRESLEEP_CYCLES)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def _bench_gemm_family(args, world, rank, group, dev, dtype, pk, row):
    from .ops import gemm as G
    M, N, K = args.m, args.n, args.k
    row.update({"m": M, "n": N, "k": K})
    G.CTA_PAIR = args.cta_pair
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
        if getattr(args, "sweep_comm", ""):
            # pusher-CTA count x tiling in one process (one heap and NCCL bring-up): extra rows before the default one
            for pair in (0, 1, 2):
                for nc in (int(x) for x in args.sweep_comm.split(",")):
                    G.CTA_PAIR, ctx.num_comm_sms = pair, nc
                    t = timed_us(lambda: G.ag_gemm_intra_node(a, b, ctx, out=c), args.iters, args.warmup, world, group)
                    if rank == 0:
                        print(json.dumps({"op": "ag_gemm_sweep", "world": world, "m": M, "n": N, "k": K, "cta_pair": pair,
                                          "num_comm_sms": nc, "us": round(t, 2)}), flush=True)
            G.CTA_PAIR, ctx.num_comm_sms = args.cta_pair, 0
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
    compute_us = flops / (pk["bf16_tflops"] * 1e6)
    row.update({"us": round(us, 2), "tflops_per_gpu": round(flops / us / 1e6, 1),
                "roofline_us": round(max(compute_us, link_us), 2),
                "roofline_fraction": round(max(compute_us, link_us) / us, 3)})
    if base is not None:
        row.update({"torch_us": round(base, 2), "speedup_vs_torch": round(base / us, 3)})


def _bench_gemm_fp8(args, world, rank, group, dev, dtype, pk, row):
    """Block-scaled fp8 GEMM / AG-GEMM. Baseline: NCCL all-gather of rows and scales +
    ``torch._scaled_mm`` with the same 1x128 / 128x128 scales when this torch build takes them, else
    the cuBLAS bf16 matmul of the same shape (named in ``baseline``)."""
    from .ops import gemm_fp8 as F
    M, N, K = args.m, args.n, args.k
    ag = args.op == "ag_gemm_fp8"
    mpr, npr = (M // world, N // world) if ag else (M, N)
    row.update({"m": M, "n": N, "k": K, "dtype": "fp8_e4m3 (1x128 / 128x128 fp32 scales) -> bf16"})
    a, sa = F.quantize_fp8_rowwise(torch.randn(mpr, K, device=dev))
    b, sb = F.quantize_fp8_blockwise(torch.randn(npr, K, device=dev) * K ** -0.5)
    c = torch.empty(M if ag else mpr, npr, device=dev, dtype=torch.bfloat16)
    if ag:
        ctx = F.create_ag_gemm_fp8_context(M, K, rank, world, device=dev, group=group)
        us = timed_us(lambda: F.ag_gemm_fp8(a, sa, b, sb, ctx, out=c), args.iters, args.warmup, world, group)
        link_us = (world - 1) * mpr * (K + K // 32) / (NVLINK_GBS * 1e3)
    else:
        us = timed_us(lambda: F.gemm_fp8_blockscaled(a, sa, b, sb, out=c), args.iters, args.warmup, 1)
        link_us = 0.0
    flops = 2.0 * c.shape[0] * npr * K
    compute_us = flops / (2.0 * pk["bf16_tflops"] * 1e6)   # dense fp8 peak = 2 x the bf16 figure
    row.update({"us": round(us, 2), "tflops_per_gpu": round(flops / us / 1e6, 1),
                "roofline_us": round(max(compute_us, link_us), 2), "roofline_fraction": round(max(compute_us, link_us) / us, 3),
                "roofline_note": "compute bound taken as 2 x the measured cuBLAS bf16 throughput"})
    if args.no_baseline:
        return
    full = torch.empty(c.shape[0], K, device=dev, dtype=torch.uint8)
    fs = torch.empty(c.shape[0], K // 128, device=dev, dtype=torch.float32)
    a16, b16 = torch.empty(c.shape[0], K, device=dev, dtype=torch.bfloat16), b.to(torch.bfloat16)

    def gather():
        if ag and world > 1:
            dist.all_gather_into_tensor(full, a.view(torch.uint8), group=group)
            dist.all_gather_into_tensor(fs, sa, group=group)
    fa = full.view(F.FP8) if ag and world > 1 else a
    fsa = fs if ag and world > 1 else sa
    name = "nccl all_gather + torch._scaled_mm (blockwise scales)"
    try:
        torch._scaled_mm(fa, b.t(), scale_a=fsa, scale_b=sb.t(), out_dtype=torch.bfloat16)

        def ref():
            gather()
            torch._scaled_mm(fa, b.t(), scale_a=fsa, scale_b=sb.t(), out_dtype=torch.bfloat16)
    except Exception:  # noqa: BLE001 - this torch build has no blockwise-scaled path on this device
        name = "nccl all_gather + cuBLAS bf16 matmul of the same shape"

        def ref():
            gather()
            torch.matmul(a16, b16.t(), out=c)
    torch.cuda.synchronize()
    base = timed_us(ref, args.iters, args.warmup, world, group)
    row.update({"baseline": name, "torch_us": round(base, 2), "speedup_vs_torch": round(base / us, 3)})


def _bench_decode(args, world, rank, group, dev, dtype, pk, row):
    """--kv = TOTAL keys per sequence (split evenly over the ranks for sp_decode)."""
    import math

    from .ops import flash_decode as FD
    B, Hq, Hkv, D, page = args.batch, args.hq, args.hkv, args.head_dim, args.page_size
    kv_local = args.kv // world
    nblk = (kv_local + page - 1) // page
    k = torch.randn(B * nblk, page, Hkv, D, device=dev, dtype=dtype)
    v = torch.randn(B * nblk, page, Hkv, D, device=dev, dtype=dtype)
    table = torch.arange(B * nblk, device=dev, dtype=torch.int32).view(B, nblk)
    q = torch.randn(B, Hq, D, device=dev, dtype=dtype)
    scale = 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    row.update({"batch": B, "hq": Hq, "hkv": Hkv, "head_dim": D, "kv_total": args.kv, "kv_per_rank": kv_local,
                "kv_split": args.kv_split if args.kv_split > 0 else FD.default_splits(B, Hkv, nblk * page, dev, D)})
    if args.op == "decode":
        lens = torch.full((B,), kv_local, dtype=torch.int32, device=dev)
        us = timed_us(lambda: FD.gqa_fwd_batch_decode(q, k, v, None, None, lens, table, scale, output_combine=out,
                                                      kv_split=args.kv_split), args.iters, args.warmup, 1)
        base = None
    else:
        glens = torch.full((world, B), kv_local, dtype=torch.int32, device=dev)
        ctx = FD.create_sp_decode_context(rank, world, B, Hq, D, group=group, device=dev)
        us = timed_us(lambda: FD.sp_gqa_fwd_batch_decode(ctx, q, k, v, glens, table, scale, out=out, kv_split=args.kv_split),
                      args.iters, args.warmup, world, group)
        base = None
        if not args.no_baseline:
            # local partial (our kernel) + NCCL all_gather + torch merge = the non-fused pipeline
            parts = torch.empty(world, B, Hq, D + 1, device=dev, dtype=torch.float32)

            def ref():
                mine = FD.gqa_fwd_batch_decode_intra_rank(q, k, v, None, None, glens[rank], table, scale)
                if world > 1:
                    dist.all_gather_into_tensor(parts, mine, group=group)
                else:
                    parts[0].copy_(mine)
                FD.inter_rank_combine(parts, dtype, out=out)
            base = timed_us(ref, args.iters, args.warmup, world, group)
    kv_bytes = 2.0 * B * kv_local * Hkv * D * 2
    hbm_us = kv_bytes / (pk["hbm_gbs"] * 1e3)
    row.update({"us": round(us, 2), "kv_gbps": round(kv_bytes / us / 1e3, 1), "roofline_us": round(hbm_us, 2),
                "roofline_fraction": round(hbm_us / us, 3)})
    if base is not None:
        row.update({"unfused_us": round(base, 2), "speedup_vs_unfused": round(base / us, 3)})


def _bench_a2a(args, world, rank, group, dev, dtype, pk, row):
    from .ops import all_to_all as A
    from .ops import moe_utils as MU
    T, H, E, K = args.tokens, args.hidden, args.experts, args.topk
    row.update({"tokens_per_rank": T, "hidden": H, "experts": E, "topk": K})
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    ids, w = MU.topk_softmax(torch.randn(T, E, device=dev), K)
    ctx = A.create_moe_dispatch_context(T, H, K, E, rank, world, group=group, device=dev)
    state = {}

    def dispatch():
        state["recv"] = A.moe_dispatch(ctx, x, ids, w)

    def both():
        # identity experts: the fp8 rows are dequantised straight into the symmetric buffer the combine reads
        rx, rs, splits = A.moe_dispatch(ctx, x, ids, w)
        A.dequant_fp8(rx, rs, out=A.moe_expert_out_buffer(ctx))
        A.moe_combine(ctx, None, splits)

    dispatch()
    A.dequant_fp8(*state["recv"][:2], out=A.moe_expert_out_buffer(ctx))
    us_d = timed_us(dispatch, args.iters, args.warmup, world, group)
    A.dequant_fp8(*state["recv"][:2], out=A.moe_expert_out_buffer(ctx))
    us_c = timed_us(lambda: A.moe_combine(ctx, None, state["recv"][2]), args.iters, args.warmup, world, group)
    us_b = timed_us(both, args.iters, args.warmup, world, group)
    # the expert-parallel layer on the same problem: bf16 rows into the expert-major compact layout, plain-sum combine
    from .models import EPAll2AllLayer
    layer = EPAll2AllLayer(group, T, H, K, rank, E, world, world, device=dev)

    def ep_both():
        rows = layer.dispatch(x, ids)
        layer.output_buffer().copy_(rows)     # identity experts
        layer.combine()
    layer.dispatch(x, ids)
    us_ed = timed_us(lambda: layer.dispatch(x, ids), args.iters, args.warmup, world, group)
    us_ec = timed_us(lambda: layer.combine(), args.iters, args.warmup, world, group)
    row.update({"ep_layer_dispatch_us": round(us_ed, 2), "ep_layer_combine_us": round(us_ec, 2)})
    del ep_both
    out_bytes = T * K * (H + H // 128 * 4) * (world - 1) / world
    back_bytes = T * K * H * 2 * (world - 1) / world
    link_us = (out_bytes + back_bytes) / (NVLINK_GBS * 1e3)
    row.update({"dispatch_us": round(us_d, 2), "combine_us": round(us_c, 2), "dispatch_dequant_combine_us": round(us_b, 2),
                "us": round(us_d + us_c, 2), "roofline_us": round(link_us, 2),
                "roofline_fraction": round(link_us / (us_d + us_c), 3)})
    if not args.no_baseline and world > 1:
        # NCCL all_to_all_single of the same payload with equal splits (bf16 both ways)
        rows = T * K // world * world
        send = torch.randn(rows, H, device=dev).to(torch.bfloat16)
        recv = torch.empty_like(send)
        base = timed_us(lambda: (dist.all_to_all_single(recv, send, group=group), dist.all_to_all_single(send, recv, group=group)),
                        args.iters, args.warmup, world, group)
        row.update({"nccl_a2a_x2_us": round(base, 2), "speedup_vs_nccl": round(base / (us_d + us_c), 3)})


def _bench_allgather(args, world, rank, group, dev, dtype, pk, row):
    from .ops import collectives as CO
    from .runtime import symm_heap
    nbytes = args.bytes // world * world
    heap = symm_heap(group)
    buf = heap.empty((nbytes,), torch.uint8)
    ctx = CO.create_fast_allgather_context(rank, 0, world, 1, max_buffer_size=nbytes, group=group, device=dev)
    row.update({"bytes": nbytes, "mode": args.mode})

    def step():
        CO.fast_allgather(buf, ctx, mode=args.mode)
        CO.barrier_all_on_stream()  # in-place buffer: nobody may start the next round early
    us = timed_us(step, args.iters, args.warmup, world, group)
    us_bar = timed_us(CO.barrier_all_on_stream, args.iters, args.warmup, world, group)
    link_us = nbytes * (world - 1) / world / (NVLINK_GBS * 1e3)
    row.update({"us": round(us - us_bar, 2), "barrier_us": round(us_bar, 2), "bus_gbps": round(nbytes * (world - 1) / world / max(us - us_bar, 1e-3) / 1e3, 1),
                "roofline_us": round(link_us, 2), "roofline_fraction": round(link_us / max(us - us_bar, 1e-3), 3)})
    if not args.no_baseline and world > 1:
        mine = torch.empty(nbytes // world, dtype=torch.uint8, device=dev)
        full = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        base = timed_us(lambda: dist.all_gather_into_tensor(full, mine, group=group), args.iters, args.warmup, world, group)
        row.update({"nccl_us": round(base, 2)})


def _bench_nvls(args, world, rank, group, dev, dtype, pk, row):
    """NVLS (multimem) collectives; needs TDIST_NVLS=1 in the environment so that the heap has a multicast
    alias. `--mode` is allgather, reduce_scatter or allreduce; baseline = the same NCCL collective."""
    from .ops import nvls as NV
    from .runtime import symm_heap
    n = args.bytes // (2 * 16 * world) * (16 * world)   # bf16 elements, segments of whole 16-byte vectors
    heap = symm_heap(group)
    buf = heap.empty((n,), torch.bfloat16)
    row.update({"bytes": n * 2, "mode": args.mode, "multicast": NV.nvls_available(buf)})
    if not NV.nvls_available(buf):
        row["error"] = "no multicast alias (run with TDIST_NVLS=1 on an NVSwitch system)"
        return
    ctx = NV.create_nvls_context(rank, world, heap=heap, group=group, device=dev)
    buf.local.normal_()
    out = torch.empty(n // world, dtype=torch.bfloat16, device=dev)
    full = torch.empty(n, dtype=torch.bfloat16, device=dev)
    if args.mode == "allgather":
        fn, ref = (lambda: NV.nvls_allgather(buf, ctx)), (lambda: dist.all_gather_into_tensor(full, out, group=group))
        wire = n * 2 * (world - 1) / world
    elif args.mode == "reduce_scatter":
        fn, ref = (lambda: NV.nvls_reduce_scatter(buf, ctx, out)), (lambda: dist.reduce_scatter_tensor(out, full, group=group))
        wire = n * 2 * (world - 1) / world
    else:
        fn, ref = (lambda: NV.nvls_allreduce(buf, ctx)), (lambda: dist.all_reduce(full, group=group))
        wire = 2 * n * 2 * (world - 1) / world
    us = timed_us(fn, args.iters, args.warmup, world, group)
    row.update({"us": round(us, 2), "bus_gbps": round(wire / us / 1e3, 1)})
    if not args.no_baseline:
        full.zero_()
        base = timed_us(ref, args.iters, args.warmup, world, group)
        row.update({"nccl_us": round(base, 2), "speedup_vs_nccl": round(base / us, 3)})


def _bench_local_collectives(args, world, rank, group, dev, dtype, pk, row):
    """The collective kernels of four emulated ranks on ONE GPU (send halves of every rank, then the receive halves, so
    no launch waits for a launch that has not run): LL all-gather, push all-gather, reduce-scatter with the fused
    top-k reduce. For single-GPU profiles of these kernels; the times include no link."""
    from .ops import collectives as CO
    from .runtime import LocalWorld
    W = 4
    lw = LocalWorld(W, dev)
    seg = max(16, args.bytes // W // 16 * 16)
    row.update({"emulated_ranks": W, "segment_bytes": seg})
    for mode in ("push2d_ll", "push2d"):
        ctxs = [CO.create_fast_allgather_context(r, 0, W, 1, max_buffer_size=W * seg, heap=lw.heap(r), device=dev) for r in range(W)]
        bufs = [lw.heap(r).empty((W * seg,), torch.uint8) for r in range(W)]

        def step():
            for r in range(W):
                CO.fast_allgather(bufs[r], ctxs[r], mode=mode, phase=1)
            for r in range(W):
                CO.fast_allgather(bufs[r], ctxs[r], mode=mode, phase=2)
        row[f"allgather_{mode}_us_per_rank"] = round(timed_us(step, args.iters, args.warmup, 1) / W, 2)
    M, N, topk = args.tokens * W, args.hidden, args.topk
    ctxs = [CO.create_reduce_scater_2d_ctx(M, N, r, W, dtype=torch.bfloat16, heap=lw.heap(r), device=dev) for r in range(W)]
    y = torch.randn(M * topk, N, device=dev).to(torch.bfloat16)
    pos = torch.randperm(M * topk, device=dev).to(torch.int32)
    w = torch.rand(M, topk, device=dev)

    def rs_step():
        for r in range(W):
            CO.topk_reduce_scatter(y, pos, w, M, topk, ctxs[r], phase=1)
        for r in range(W):
            CO.topk_reduce_scatter(y, pos, w, M, topk, ctxs[r], phase=2)
    row["topk_reduce_scatter_us_per_rank"] = round(timed_us(rs_step, args.iters, args.warmup, 1) / W, 2)


def _bench_moe_route(args, world, rank, group, dev, dtype, pk, row):
    """The MoE routing kernels on one GPU: softmax + top-k, stable expert sort, block-aligned rank-major sort."""
    from .ops import moe_utils as MU
    T, E, K = args.tokens, args.experts, args.topk
    logits = torch.randn(T, E, device=dev)
    ids, _ = MU.topk_softmax(logits, K)
    row.update({"tokens": T, "experts": E, "topk": K})
    row["topk_softmax_us"] = round(timed_us(lambda: MU.topk_softmax(logits, K), args.iters, args.warmup, 1), 2)
    row["route_us"] = round(timed_us(lambda: MU.route(ids, E), args.iters, args.warmup, 1), 2)
    ranks = 8 if T % 8 == 0 else 1
    row["align_block_size_us"] = round(timed_us(lambda: MU.sort_topk_ids_align_block_size(ids, E, ranks, T // ranks, 128),
                                                args.iters, args.warmup, 1), 2)


def _bench_moe_tp(args, world, rank, group, dev, dtype, pk, row):
    """Tensor-parallel MoE (Mixtral-like by default: 8192 tokens, hidden 4096, intermediate 14336, 8 experts, top-2):
    AllGather + GroupGEMM and GroupGEMM + top-k reduce + ReduceScatter, fused against staged."""
    from .ops import moe_tp as MT
    M, H, I, E, topk = args.m, args.k, args.n, args.experts, args.topk
    mpr = M // world
    row.update({"tokens": M, "hidden": H, "intermediate": I, "experts": E, "topk": topk})
    gen = torch.Generator(device=dev).manual_seed(0)
    ids = torch.randint(0, E, (M, topk), device=dev, generator=gen).to(torch.int32)
    if world > 1:
        dist.broadcast(ids, 0, group=group)
    w = torch.rand(M, topk, device=dev, generator=gen)
    a = torch.randn(mpr, H, device=dev, dtype=dtype)
    b1 = (torch.randn(E, H, I // world, device=dev) * H ** -0.5).to(dtype)
    ctx1 = MT.create_ag_group_gemm_intra_node_context(group, a, b1, ids, E, max_M=M, rank=rank, num_ranks=world)
    h = torch.randn(M * topk, I // world, device=dev, dtype=dtype)
    b2 = (torch.randn(E, I // world, H, device=dev) * I ** -0.5).to(dtype)
    ctx2 = MT.create_moe_rs_context(group, rank, world, world, M, H, E, topk, dtype, dtype, dev, full_topk_ids=ids, full_topk_weight=w)
    flops1 = 2.0 * M * topk * (I // world) * H
    # fused: one grouped-GEMM launch that stages its rows block by block (its own warps), waits per block for the
    # all-gather, stores every row at its final position; top-k reduce inside the reduce-scatter.
    # staged: all-gather, row-gather, grouped GEMM, un-sort, top-k reduce, reduce-scatter as separate launches.
    for name, mode, flag in (("fused", "fused", True), ("staged", "staged", False)):
        MT.AG_GROUP_GEMM_MODE = mode
        MT.FUSED_TOPK_RS = flag
        us1 = timed_us(lambda: MT.ag_group_gemm_intra_node(a, b1, ctx1), args.iters, args.warmup, world, group)
        us2 = timed_us(lambda: MT.moe_reduce_rs(rank, world, world, h, b2, ctx2), args.iters, args.warmup, world, group)
        row.update({f"ag_group_gemm_{name}_us": round(us1, 1), f"moe_reduce_rs_{name}_us": round(us2, 1),
                    f"ag_group_gemm_{name}_tflops": round(flops1 / us1 / 1e6, 1), f"moe_reduce_rs_{name}_tflops": round(flops1 / us2 / 1e6, 1)})
    MT.AG_GROUP_GEMM_MODE, MT.FUSED_TOPK_RS = "fused", True
    row["ag_group_gemm_fused_over_staged"] = round(row["ag_group_gemm_staged_us"] / row["ag_group_gemm_fused_us"], 3)
    row["moe_reduce_rs_fused_over_staged"] = round(row["moe_reduce_rs_staged_us"] / row["moe_reduce_rs_fused_us"], 3)


def _bench_fused_local(args, world, rank, group, dev, dtype, pk, row):
    """One rank's fused AG-GEMM and GEMM-RS kernels on ONE GPU, against peer buffers prepared by the host (the
    other ranks of a 2-rank world are emulated in the same process). The kernels run their real code paths: pusher
    CTAs storing into the peer's workspace, flag waits, epilogue stores into the peer's staging, reduce tail. Meant
    for single-process profilers; the timings are of this one launch, not of a collective step."""
    from .ops import gemm as G
    from .runtime import LocalWorld
    W = 2
    M, N, K = args.m, args.n, args.k
    mpr = M // W
    row.update({"m": M, "n": N, "k": K, "emulated_world": W})
    lw = LocalWorld(W, dev)
    A = [torch.randn(mpr, K, device=dev, dtype=dtype) for _ in range(W)]
    B = [(torch.randn(N // W, K, device=dev) * K ** -0.5).to(dtype) for _ in range(W)]
    ctxs = [G.create_ag_gemm_intra_node_context(A[r], B[r], r, W, max_M=M, heap=lw.heap(r)) for r in range(W)]
    mt = (mpr + 127) // 128
    times = {}
    for it in range(args.warmup + 1):
        ctx = ctxs[0]
        half = (ctx.epoch + 1) & 1
        ws = ctx.workspace.local[half][: W * mpr * K].view(W, mpr, K)
        ws[1].copy_(A[1])                                    # rank 1's rows "arrive", with their flags
        ctx.flags.local[half][: W * mt].view(W, mt)[1].fill_(ctx.epoch + 1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        c = G.ag_gemm_intra_node(A[0], B[0], ctx)
        e1.record()
        torch.cuda.synchronize()
        times["ag_gemm_rank0_us"] = round(e0.elapsed_time(e1) * 1e3, 1)
    ref = torch.cat(A).float() @ B[0].float().t()
    row["ag_max_err"] = float((c.float() - ref).abs().max())
    # GEMM-RS: rank 0's kernel; rank 1's partial tiles and flags are written by the host
    kl = K // W
    X = [torch.randn(M, kl, device=dev, dtype=dtype) for _ in range(W)]
    V = [(torch.randn(N, kl, device=dev) * K ** -0.5).to(dtype) for _ in range(W)]
    rctx = G.create_gemm_rs_context(M, N, 0, W, output_dtype=dtype, heap=lw.heap(0), device=dev)
    G.create_gemm_rs_context(M, N, 1, W, output_dtype=dtype, heap=lw.heap(1), device=dev)   # the peer's half of the symmetric state
    partial1 = (X[1].float() @ V[1].float().t())[:mpr].to(dtype)
    tiles = mt * ((N + 255) // 256)
    for it in range(args.warmup + 1):
        half = (rctx.epoch + 1) & 1
        rctx.staging.local[half][: W * mpr * N].view(W, mpr, N)[1].copy_(partial1)
        rctx.flags.local[half][: tiles * W].view(tiles, W)[:, 1].fill_(rctx.epoch + 1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        o = G.gemm_rs(X[0], V[0], rctx)
        e1.record()
        torch.cuda.synchronize()
        times["gemm_rs_rank0_us"] = round(e0.elapsed_time(e1) * 1e3, 1)
    ref = (X[0].float() @ V[0].float().t() + X[1].float() @ V[1].float().t())[:mpr]
    row["rs_max_err"] = float((o.float() - ref).abs().max())
    row.update(times)


def _run_suite(args, world, rank, group, dev, dtype, pk):
    """Every headline configuration in one process (one NCCL / heap bring-up): the two tensor-parallel
    GEMMs on the m8192 n49152 k12288 problem, MoE dispatch+combine (128 tokens, hidden 7168, 256 experts,
    top-8), sequence-parallel decode (32/8 heads, D 128, batch 1 and 8, 32K / 128K / 1M keys in total),
    and the all-gather modes at 64 KB and 16 MB."""
    import copy
    global PRESLEEP_CYCLES

    def emit(row):
        if rank == 0:
            print(json.dumps(row), flush=True)

    def run(op, fn, **over):
        a = copy.copy(args)
        a.op = op
        for k, v in over.items():
            setattr(a, k, v)
        row = {"op": op, "world": world, "dtype": a.dtype, "peaks": pk["source"]}
        try:
            fn(a, world, rank, group, dev, dtype, pk, row)
        except Exception as e:  # noqa: BLE001 - keep the rest of the suite alive
            row["error"] = repr(e)[:300]
        emit(row)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()

    PRESLEEP_CYCLES = 0
    run("ag_gemm", _bench_gemm_family, m=8192, n=49152, k=12288)
    run("gemm_rs", _bench_gemm_family, m=8192, n=12288, k=49152)
    run("ag_gemm_fp8", _bench_gemm_fp8, m=8192, n=49152, k=12288)
    # the shapes of the reference's published intra-node charts (speed-up over PyTorch + NCCL on 8 x H800)
    for (n, k) in ((11008, 4096), (14336, 4096), (28672, 8192), (53248, 16384), (29568, 8192)):
        run("ag_gemm", _bench_gemm_family, m=8192, n=n, k=k)
    for (n, k) in ((4096, 11008), (4096, 14336), (3584, 14336), (4608, 36864), (8192, 28672), (8192, 29568)):
        run("gemm_rs", _bench_gemm_family, m=8192, n=n, k=k)
    # tensor-parallel MoE (8 experts, top-2, hidden 4096, intermediate 14336 split over the ranks): one-launch against staged
    run("moe_tp", _bench_moe_tp, m=8192, n=14336, k=4096, experts=8, topk=2, iters=10)
    run("moe_tp", _bench_moe_tp, m=2048, n=14336, k=4096, experts=8, topk=2, iters=20)
    PRESLEEP_CYCLES = int(30 * 1.9e6)
    if world > 1 or True:
        run("a2a", _bench_a2a, tokens=128, hidden=7168, experts=256, topk=8, iters=50)
    for batch in (1, 8):
        for kv in (32768, 131072, 1048576):
            run("sp_decode", _bench_decode, batch=batch, kv=kv, hq=32, hkv=8, head_dim=128, iters=30)
    if world > 1:
        for mode in ("pull", "push2d", "push_ordered", "push2d_ll"):
            for nbytes in (65536, 16 << 20):
                run("allgather", _bench_allgather, mode=mode, bytes=nbytes, iters=30)
        if os.environ.get("TDIST_NVLS", "0") == "1":
            for mode in ("allgather", "reduce_scatter", "allreduce"):
                for nbytes in (65536, 16 << 20, 256 << 20):
                    run("nvls", _bench_nvls, mode=mode, bytes=nbytes, iters=30)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["gemm", "ag_gemm", "gemm_rs", "gemm_fp8", "ag_gemm_fp8", "decode", "sp_decode", "a2a", "allgather", "nvls", "nvls_suite", "moe_tp", "fused_local", "local_collectives", "moe_route", "suite"])
    ap.add_argument("--shape", default="", help="MxNxK in one argument (torchrun swallows a bare --m)")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=12288)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--kv", type=int, default=131072, help="total keys per sequence")
    ap.add_argument("--kv-split", type=int, default=-1, help="decode: CTAs per (batch, kv head); -1 = the launcher's heuristic")
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--bytes", type=int, default=1 << 20)
    ap.add_argument("--mode", default="push2d")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--cta-pair", type=int, default=-1)
    ap.add_argument("--no-baseline", action="store_true")
    ap.add_argument("--sweep-comm", default="", help="ag_gemm: comma-separated pusher-CTA counts to time under both pair tilings")
    ap.add_argument("--presleep-ms", type=float, default=-1.0,
                    help="spin the GPU this long before each timed loop (default: 30 ms for the latency ops, 0 for GEMMs)")
    args = ap.parse_args(argv)
    global PRESLEEP_CYCLES
    if args.shape:
        args.m, args.n, args.k = (int(v) for v in args.shape.lower().split("x"))
    if args.presleep_ms < 0:
        args.presleep_ms = 0.0 if args.op in ("gemm", "ag_gemm", "gemm_rs", "gemm_fp8", "ag_gemm_fp8", "moe_tp", "fused_local") else 30.0
    PRESLEEP_CYCLES = int(args.presleep_ms * 1.9e6)

    from .runtime import check_status, finalize_distributed, initialize_distributed

    world = int(os.environ.get("WORLD_SIZE", "1"))
    group = initialize_distributed(seed=0) if world > 1 or "RANK" in os.environ else None
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    pk = peaks()
    row = {"op": args.op, "world": world, "dtype": args.dtype, "peaks": pk["source"]}
    if args.op == "nvls_suite":
        import copy
        for mode in ("allgather", "reduce_scatter", "allreduce"):
            for nbytes in (65536, 16 << 20, 256 << 20):
                a2 = copy.copy(args)
                a2.op, a2.mode, a2.bytes = "nvls", mode, nbytes
                r2 = {"op": "nvls", "world": world, "dtype": "bf16", "peaks": pk["source"]}
                try:
                    _bench_nvls(a2, world, rank, group, dev, dtype, pk, r2)
                except Exception as e:  # noqa: BLE001 - keep the other rows
                    r2["error"] = repr(e)[:300]
                if rank == 0:
                    print(json.dumps(r2), flush=True)
        check_status()
        if dist.is_initialized():
            finalize_distributed()
        return 0
    if args.op == "suite":
        _run_suite(args, world, rank, group, dev, dtype, pk)
        check_status()
        if dist.is_initialized():
            finalize_distributed()
        return 0
    if args.op in ("gemm", "ag_gemm", "gemm_rs"):
        _bench_gemm_family(args, world, rank, group, dev, dtype, pk, row)
    elif args.op in ("gemm_fp8", "ag_gemm_fp8"):
        _bench_gemm_fp8(args, world, rank, group, dev, dtype, pk, row)
    elif args.op in ("decode", "sp_decode"):
        _bench_decode(args, world, rank, group, dev, dtype, pk, row)
    elif args.op == "a2a":
        _bench_a2a(args, world, rank, group, dev, dtype, pk, row)
    elif args.op == "nvls":
        _bench_nvls(args, world, rank, group, dev, dtype, pk, row)
    elif args.op == "fused_local":
        _bench_fused_local(args, world, rank, group, dev, dtype, pk, row)
    elif args.op == "moe_tp":
        if args.experts == 256 and args.topk == 8 and args.n == 6144 and args.k == 12288:   # untouched defaults: Mixtral-like
            args.n, args.k, args.experts, args.topk = 14336, 4096, 8, 2
        _bench_moe_tp(args, world, rank, group, dev, dtype, pk, row)
    elif args.op == "local_collectives":
        _bench_local_collectives(args, world, rank, group, dev, dtype, pk, row)
    elif args.op == "moe_route":
        _bench_moe_route(args, world, rank, group, dev, dtype, pk, row)
    else:
        _bench_allgather(args, world, rank, group, dev, dtype, pk, row)
    check_status()
    if rank == 0:
        print(json.dumps(row), flush=True)
    if dist.is_initialized():
        finalize_distributed()
    return 0


if __name__ == "__main__":
    sys.exit(main())
