"""Block-scaled fp8 (e4m3) GEMM and fused AllGather-GEMM (``csrc/kernels/gemm_fp8_sm100.cu``).

Scale layout (the DeepSeek-V3 one): activations carry one fp32 scale per row per 128 values of K
(``sa[M, K/128]``), weights one per 128 x 128 block (``sb[ceil(N/128), K/128]``); the product is
accumulated in fp32 and written as bf16:

    C[m, n] = sum_kb sa[m, kb] * sb[n // 128, kb] * dot(A[m, kb-th block], B[n, kb-th block])

* ``quantize_fp8_rowwise(x) -> (x_fp8, sa)`` and ``quantize_fp8_blockwise(w) -> (w_fp8, sb)``
* ``gemm_fp8_blockscaled(a, sa, b, sb) -> bf16 [M, N]``
* ``create_ag_gemm_fp8_context`` / ``ag_gemm_fp8(a, sa, b, sb, ctx) -> bf16 [M, N/ws]``: the gather of
  the fp8 rows and of their scales runs inside the GEMM kernel (pusher CTAs + per-block flags).

The reference runs AG-GEMM on fp8 inputs without scales (its test
python/triton_dist/test/nvidia/test_ag_gemm.py takes ``--dtype float8_e4m3fn``) and quantises
activations to this 1x128 layout in its all-to-all tutorial (tutorials/04-deepseek-infer-all2all.py).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import _lib
from ..utils.profile import nvtx_range
from ..runtime import SymmTensor, default_timeout_ns, global_status, symm_heap

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
launch_count = 0


def _cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def quantize_fp8_rowwise(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[M, K] -> (e4m3 [M, K], fp32 scales [M, K/128]); value = fp8 * scale."""
    M, K = x.shape
    if K % 128:
        raise ValueError("K must be a multiple of 128")
    xb = x.float().view(M, K // 128, 128)
    amax = xb.abs().amax(dim=2).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (xb / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).to(FP8).view(M, K)
    return q, scale.contiguous()


def quantize_fp8_blockwise(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[N, K] -> (e4m3 [N, K], fp32 scales [ceil(N/128), K/128]); one scale per 128 x 128 block."""
    N, K = w.shape
    if K % 128:
        raise ValueError("K must be a multiple of 128")
    nb = _cdiv(N, 128)
    wp = torch.zeros((nb * 128, K), dtype=torch.float32, device=w.device)
    wp[:N] = w.float()
    blocks = wp.view(nb, 128, K // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(nb * 128, K)[:N].to(FP8)
    return q.contiguous(), scale.contiguous()


def dequantize_fp8(a: torch.Tensor, sa: torch.Tensor, block_rows: int = 1) -> torch.Tensor:
    """fp32 values of a block-scaled fp8 tensor (``block_rows`` 1 for activations, 128 for weights)."""
    rows, K = a.shape
    s = sa.repeat_interleave(block_rows, dim=0)[:rows] if block_rows > 1 else sa
    return a.float() * s.repeat_interleave(128, dim=1)


def gemm_fp8_reference(a, sa, b, sb) -> torch.Tensor:
    """The op restated in fp32 torch: the oracle of the GPU tests and the CPU path."""
    return (dequantize_fp8(a, sa, 1) @ dequantize_fp8(b, sb, 128).t()).to(torch.bfloat16)


def _check(a, sa, b, sb):
    if a.dtype != FP8 or b.dtype != FP8:
        raise TypeError("fp8 GEMM operands must be torch.float8_e4m3fn")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1] or a.shape[1] % 128:
        raise ValueError(f"expected a[M,K], b[N,K] with K a multiple of 128, got {tuple(a.shape)} and {tuple(b.shape)}")
    if b.shape[0] % 8:
        raise ValueError("N must be a multiple of 8")
    kb = a.shape[1] // 128
    if tuple(sa.shape) != (a.shape[0], kb) or tuple(sb.shape) != (_cdiv(b.shape[0], 128), kb):
        raise ValueError(f"scale shapes {tuple(sa.shape)} / {tuple(sb.shape)} do not match the operands")
    if sa.dtype != torch.float32 or sb.dtype != torch.float32:
        raise TypeError("scales must be fp32")
    for t in (a, sa, b, sb):
        if not t.is_contiguous():
            raise ValueError("fp8 GEMM operands and scales must be contiguous")


def _base(a, sa, b, sb, world, rank, mode) -> "_lib.GemmFp8Args":
    g = _lib.GemmFp8Args()
    g.a, g.sa, g.b, g.sb = a.data_ptr(), sa.data_ptr(), b.data_ptr(), sb.data_ptr()
    g.n, g.k = b.shape[0], a.shape[1]
    g.world, g.rank, g.mode = world, rank, mode
    st = global_status()
    g.status = st.device_ptr if st is not None else None
    g.timeout_ns = default_timeout_ns()
    g.stream = torch.cuda.current_stream(a.device).cuda_stream
    return g


def _launch(g) -> None:
    global launch_count
    _lib.check(_lib.lib().tdist_gemm_fp8_run(C.byref(g)), "tdist_gemm_fp8_run")
    launch_count += 1


@nvtx_range("tdist.gemm_fp8_blockscaled")
def gemm_fp8_blockscaled(a: torch.Tensor, sa: torch.Tensor, b: torch.Tensor, sb: torch.Tensor,
                         out: Optional[torch.Tensor] = None, num_sms: int = 0) -> torch.Tensor:
    if a.device.type != "cuda":
        return gemm_fp8_reference(a, sa, b, sb)
    _check(a, sa, b, sb)
    c = out if out is not None else torch.empty((a.shape[0], b.shape[0]), dtype=torch.bfloat16, device=a.device)
    g = _base(a, sa, b, sb, 1, 0, _lib.GEMM_PLAIN)
    g.c = c.data_ptr()
    g.m_per_rank = a.shape[0]
    g.epoch = 1
    g.num_sms = num_sms
    _launch(g)
    return c


@dataclass
class AGGemmFp8Context:
    """Symmetric state of the fp8 AllGather-GEMM: double-buffered gather workspaces for rows and for
    their scales, per-128-row-block flags, and the call counter the flags carry."""

    rank: int
    world: int
    max_m_per_rank: int
    k: int
    group: object = None
    workspace: Optional[SymmTensor] = None
    scale_ws: Optional[SymmTensor] = None
    flags: Optional[SymmTensor] = None
    epoch: int = 0
    num_comm_sms: int = 0
    num_sms: int = 0


def create_ag_gemm_fp8_context(max_M: int, K: int, rank: int, num_ranks: int, device="cuda", heap=None, group=None,
                               num_comm_sms: int = 0) -> AGGemmFp8Context:
    max_mpr = _cdiv(max_M, num_ranks)
    ctx = AGGemmFp8Context(rank=rank, world=num_ranks, max_m_per_rank=max_mpr, k=K, group=group, num_comm_sms=num_comm_sms)
    if torch.device(device).type == "cuda" and num_ranks > 1:
        heap = heap or symm_heap(group)
        ctx.workspace = heap.empty((2, num_ranks * max_mpr * K), torch.uint8)
        ctx.scale_ws = heap.empty((2, num_ranks * max_mpr * (K // 128)), torch.float32)
        ctx.flags = heap.zeros((2, num_ranks * _cdiv(max_mpr, 128)), torch.int32)
    return ctx


@nvtx_range("tdist.ag_gemm_fp8")
def ag_gemm_fp8(a: torch.Tensor, sa: torch.Tensor, b: torch.Tensor, sb: torch.Tensor, ctx: AGGemmFp8Context,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``allgather(a) @ b.T`` with block scales: ``a`` / ``sa`` are this rank's ``[M/ws, K]`` rows and
    their scales, ``b`` / ``sb`` this rank's ``[N/ws, K]`` weight shard; returns bf16 ``[M, N/ws]``."""
    mpr, K = a.shape
    if a.device.type != "cuda":
        if ctx.world > 1:
            full = torch.empty((ctx.world * mpr, K), dtype=torch.uint8)
            dist.all_gather_into_tensor(full, a.view(torch.uint8).contiguous(), group=ctx.group)
            fs = torch.empty((ctx.world * mpr, K // 128), dtype=torch.float32)
            dist.all_gather_into_tensor(fs, sa.contiguous(), group=ctx.group)
            return gemm_fp8_reference(full.view(FP8), fs, b, sb)
        return gemm_fp8_reference(a, sa, b, sb)
    _check(a, sa, b, sb)
    if mpr > ctx.max_m_per_rank or K != ctx.k:
        raise ValueError(f"shard {tuple(a.shape)} exceeds the context (max rows {ctx.max_m_per_rank}, K {ctx.k})")
    c = out if out is not None else torch.empty((ctx.world * mpr, b.shape[0]), dtype=torch.bfloat16, device=a.device)
    g = _base(a, sa, b, sb, ctx.world, ctx.rank, _lib.GEMM_AG)
    g.c = c.data_ptr()
    g.m_per_rank = mpr
    ctx.epoch += 1
    g.epoch = ctx.epoch
    g.num_sms = ctx.num_sms
    g.num_comm_sms = ctx.num_comm_sms
    if ctx.world > 1:
        half = ctx.epoch & 1
        g.a_ws = ctx.workspace.local[half].data_ptr()
        g.a_ws_peer = ctx.workspace.half_ptr_arrays()[half]
        g.sa_ws = ctx.scale_ws.local[half].data_ptr()
        g.sa_ws_peer = ctx.scale_ws.half_ptr_arrays()[half]
        g.flags = ctx.flags.local[half].data_ptr()
        g.flags_peer = ctx.flags.half_ptr_arrays()[half]
    _launch(g)
    return c
