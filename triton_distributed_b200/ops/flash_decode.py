"""GQA flash decode over a paged KV cache, single-rank and sequence-parallel.

Public surface (argument conventions of the reference, kernels/nvidia/flash_decode.py:763-1004):

* ``gqa_fwd_batch_decode(q[B,Hq,D], k_cache[blocks,page,Hkv,D], v_cache, workspace, q_lens, kv_lens[B],
  block_table[B,max_blocks], scale, soft_cap=0.0, ...) -> [B,Hq,D]``
* ``gqa_fwd_batch_decode_intra_rank(...) -> fp32 [B,Hq,D+1]`` (last column = log-sum-exp), the per-rank
  partial of a sequence-parallel decode
* ``gqa_fwd_batch_decode_persistent`` — same kernel (the split merge is always fused)
* ``inter_rank_combine(partials[R,B,Hq,D+1]) -> [B,Hq,D]``
  (reference ``kernel_inter_rank_gqa_fwd_batch_decode_combine_kv``, flash_decode.py:481-532)
* ``SpDecodeContext`` / ``sp_gqa_fwd_batch_decode`` — the whole distributed step in one launch per rank:
  partial attention, split merge, exchange of O||LSE with every rank over NVLink, final merge.

CPU tensors run ``ref_paged_attn`` (a plain torch statement, also the test oracle; the reference's
own oracle is test/nvidia/test_sp_decode_attn.py:81-131).
"""
from __future__ import annotations

import ctypes as C
import math
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib
from ..utils.profile import nvtx_range
from ..runtime import SymmTensor, default_timeout_ns, global_status, symm_heap

launch_count = 0
_DTYPES = {torch.bfloat16: _lib.DT_BF16, torch.float16: _lib.DT_F16}
_SM_COUNT = {}


def _sm_count(device) -> int:
    if getattr(device, "type", "cuda") != "cuda":
        return 148   # planning on a host without a GPU: the B200's SM count
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def ref_paged_attn(q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap: float = 0.0, return_lse: bool = False):
    """fp32 reference: for every sequence gather its pages, softmax(q k^T * scale) v per head group."""
    B, Hq, D = q.shape
    _, page, Hkv, _ = k_cache.shape
    G = Hq // Hkv
    out = torch.zeros(B, Hq, D, dtype=torch.float32, device=q.device)
    lse = torch.full((B, Hq), float("-inf"), dtype=torch.float32, device=q.device)
    for b in range(B):
        n = int(kv_lens[b])
        if n == 0:
            continue
        nblk = (n + page - 1) // page
        pages = block_table[b, :nblk].long()
        k = k_cache[pages].reshape(-1, Hkv, D)[:n].float()
        v = v_cache[pages].reshape(-1, Hkv, D)[:n].float()
        qq = q[b].float().view(Hkv, G, D)
        s = torch.einsum("hgd,nhd->hgn", qq, k) * scale
        if soft_cap > 0:
            s = soft_cap * torch.tanh(s / soft_cap)
        lse[b] = torch.logsumexp(s, dim=-1).view(Hq)
        out[b] = torch.einsum("hgn,nhd->hgd", torch.softmax(s, dim=-1), v).reshape(Hq, D)
    return (out, lse) if return_lse else out


def ref_lse_merge(parts: torch.Tensor) -> torch.Tensor:
    """parts [R, ..., D+1] (O || LSE) -> merged O [..., D] in fp32."""
    o, lse = parts[..., :-1].float(), parts[..., -1].float()
    m = lse.max(dim=0).values
    w = torch.exp(lse - torch.where(torch.isinf(m), torch.zeros_like(m), m))
    w = torch.where(torch.isinf(lse) & (lse < 0), torch.zeros_like(w), w)
    den = w.sum(0).clamp_min(1e-38)
    return (o * w.unsqueeze(-1)).sum(0) / den.unsqueeze(-1)


def default_splits(B: int, Hkv: int, max_kv: int, device, head_dim: int = 128) -> int:
    """Enough (batch, kv head, split) CTAs for one wave of the machine (two CTAs fit an SM up to
    head_dim 128), but at least 256 tokens each: below that the merge of the splits (a round trip through global
    memory per eight of them) costs more than the shorter KV loop saves (batch 1, 8 kv heads, 4096 keys: 12.4 us with
    16 splits, 16.5 us with 37, 21.0 us with 64)."""
    per_sm = 2 if head_dim <= 128 else 1
    want = max(1, per_sm * _sm_count(device) // max(1, B * Hkv))
    cap = max(1, (max_kv + 255) // 256)
    return max(1, min(want, cap, 256))


class _Workspace:
    """Split-merge scratch, cached per (device, shape)."""

    cache = {}

    @classmethod
    def get(cls, device, B, Hq, Hkv, D, splits):
        key = (device, B, Hq, Hkv, D, splits)
        ws = cls.cache.get(key)
        if ws is None:
            ws = (torch.empty((B, Hq, splits, D + 2), dtype=torch.float32, device=device),
                  torch.zeros(B * Hkv, dtype=torch.int32, device=device))
            cls.cache[key] = ws
        return ws


def _launch(q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap, out, mode, splits, max_kv=None,
            ll_ptrs=None, world=1, rank=0, epoch=0, workspace=None, stream=None, push_only=False,
            ll_ptrs_odd=None, epoch_dev=None, ll_mc=None, ll_mc_odd=None):
    global launch_count
    B, Hq, D = q.shape
    blocks, page, Hkv, Dk = k_cache.shape
    if Dk != D or v_cache.shape != k_cache.shape:
        raise ValueError("flash decode needs k and v caches of the same shape with head_dim == q's")
    if q.dtype not in _DTYPES or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise TypeError("q, k_cache and v_cache must share one of bf16 / fp16")
    if not q.is_contiguous() or k_cache.stride(3) != 1 or v_cache.stride() != k_cache.stride():
        raise ValueError("q must be contiguous; caches must have a contiguous head dimension and equal strides")
    if splits <= 0:
        if max_kv is None:
            max_kv = page * block_table.shape[1]
        splits = default_splits(B, Hkv, max_kv, q.device, D)
    partial, counters = workspace if workspace is not None else _Workspace.get(q.device, B, Hq, Hkv, D, splits)
    a = _lib.DecodeArgs()
    a.q, a.k_cache, a.v_cache = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
    bt = block_table if block_table.dtype == torch.int32 else block_table.to(torch.int32)
    kl = kv_lens if kv_lens.dtype == torch.int32 else kv_lens.to(torch.int32)
    # named locals: the (possibly copied) index tensors must outlive the launch call below
    bt_c, kl_c = bt.contiguous(), kl.contiguous()
    a.block_table, a.kv_lens = bt_c.data_ptr(), kl_c.data_ptr()
    a.partial, a.counters, a.out = partial.data_ptr(), counters.data_ptr(), out.data_ptr()
    a.B, a.Hq, a.Hkv, a.head_dim, a.page_size = B, Hq, Hkv, D, page
    a.max_blocks, a.splits = bt.shape[1], splits
    a.stride_block, a.stride_token, a.stride_head = k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
    a.scale, a.soft_cap = float(scale), float(soft_cap)
    a.mode, a.dtype, a.world, a.rank, a.epoch = mode, _DTYPES[q.dtype], world, rank, epoch
    a.push_only = int(push_only)
    if ll_ptrs is not None:
        a.ll_peer = ll_ptrs
    if ll_mc is not None:
        a.ll_mc = ll_mc
        a.ll_mc_alt = ll_mc_odd
    if epoch_dev is not None:       # call number kept on the device: the launch can be captured and replayed
        a.ll_peer_alt = ll_ptrs_odd
        a.epoch_ptr = epoch_dev.data_ptr()
        a.epoch_done = epoch_dev.data_ptr() + 4
    st = global_status()
    a.status = st.device_ptr if st is not None else None
    a.timeout_ns = default_timeout_ns()
    a.stream = (stream or torch.cuda.current_stream(q.device)).cuda_stream
    if stream is not None:
        # copies made on the current stream are read on `stream`: order the two, and keep the allocator from
        # handing the copies' memory out again before `stream` is done with them
        cur = torch.cuda.current_stream(q.device)
        if stream != cur and (bt_c is not block_table or kl_c is not kv_lens):
            stream.wait_stream(cur)
        for t in (bt_c, kl_c):
            t.record_stream(stream)
    _lib.check(_lib.lib().tdist_flash_decode(C.byref(a)), "tdist_flash_decode")
    launch_count += 1
    return out


@nvtx_range("tdist.gqa_fwd_batch_decode")
def gqa_fwd_batch_decode(q, k_cache, v_cache, workspace=None, q_lens=None, kv_lens=None, block_table=None, scale=None,
                         soft_cap: float = 0.0, output_split=None, output_combine=None, kv_split: int = -1):
    """Decode attention of one query token per sequence. Returns ``[B, Hq, D]`` in q's dtype."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if q.device.type != "cuda":
        return ref_paged_attn(q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap).to(q.dtype)
    out = output_combine if output_combine is not None else torch.empty_like(q)
    return _launch(q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap, out, 0, kv_split)


gqa_fwd_batch_decode_persistent = gqa_fwd_batch_decode


def _on_stream(stream, fn, *args, **kwargs):
    """Run ``fn`` with ``stream`` (a torch stream, a raw ``cudaStream_t`` value, or None) as the current stream."""
    if stream is None or not torch.cuda.is_available():
        return fn(*args, **kwargs)
    if isinstance(stream, int):
        stream = torch.cuda.ExternalStream(stream)
    with torch.cuda.stream(stream):
        return fn(*args, **kwargs)


# The reference's AOT-compiled entry points (kernels/nvidia/flash_decode.py `*_aot`): the same calls with the stream as
# the leading argument. Kernels here are always compiled ahead of time, so they are thin wrappers.
def gqa_fwd_batch_decode_aot(stream, q, k_cache, v_cache, *args, **kwargs):
    return _on_stream(stream, gqa_fwd_batch_decode, q, k_cache, v_cache, *args, **kwargs)


def gqa_fwd_batch_decode_persistent_aot(stream, q, k_cache, v_cache, *args, **kwargs):
    return _on_stream(stream, gqa_fwd_batch_decode, q, k_cache, v_cache, *args, **kwargs)


def gqa_fwd_batch_decode_intra_rank_aot(stream, q, k_cache, v_cache, *args, **kwargs):
    return _on_stream(stream, gqa_fwd_batch_decode_intra_rank, q, k_cache, v_cache, *args, **kwargs)


def gqa_fwd_batch_decode_intra_rank(q, k_cache, v_cache, workspace=None, q_lens=None, kv_lens=None, block_table=None,
                                    scale=None, soft_cap: float = 0.0, output_split=None, output_combine=None,
                                    kv_split: int = -1):
    """Partial decode over this rank's KV shard: fp32 ``[B, Hq, D+1]``, last column = natural-log
    sum-exp (``-inf`` when the shard is empty)."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    B, Hq, D = q.shape
    if q.device.type != "cuda":
        o, lse = ref_paged_attn(q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap, return_lse=True)
        return torch.cat([o, lse.unsqueeze(-1)], dim=-1)
    out = output_combine if output_combine is not None else torch.empty((B, Hq, D + 1), dtype=torch.float32, device=q.device)
    return _launch(q, k_cache, v_cache, kv_lens, block_table, scale, soft_cap, out, 1, kv_split)


def inter_rank_combine(partials: torch.Tensor, out_dtype=torch.bfloat16, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Merge per-rank partials fp32 ``[R, B, Hq, D+1]`` into ``[B, Hq, D]``."""
    global launch_count
    R, B, Hq, D1 = partials.shape
    D = D1 - 1
    if partials.device.type != "cuda":
        return ref_lse_merge(partials).to(out_dtype)
    parts = partials.float().contiguous()
    o = out if out is not None else torch.empty((B, Hq, D), dtype=out_dtype, device=partials.device)
    _lib.check(_lib.lib().tdist_lse_combine(parts.data_ptr(), R, B * Hq, D, o.data_ptr(), _DTYPES[o.dtype],
                                            torch.cuda.current_stream(parts.device).cuda_stream), "tdist_lse_combine")
    launch_count += 1
    return o


# ---------------------------------------------------------------------------- sequence-parallel
@dataclass
class SpDecodeContext:
    """Symmetric gather buffers (two parities of LL packets) of the fused sequence-parallel decode."""

    rank: int
    world: int
    max_batch: int
    Hq: int
    head_dim: int
    gather: Optional[SymmTensor] = None   # uint8 [2, world * max_batch * Hq * (D+2)/2 * 16]
    epoch: int = 0
    group: object = None
    # With `device_epoch` the call number lives in device memory (int32 [2]: last completed call, scratch) and the
    # kernel advances it itself, so a captured launch stays valid on replay. Every rank must choose the same way.
    epoch_dev: Optional[torch.Tensor] = None


# the sequence-parallel exchange through the NVSwitch multicast alias when the heap has one (TDIST_NVLS=1);
# TDIST_SP_DECODE_NVLS=0 keeps the per-rank stores
SP_DECODE_NVLS = os.environ.get("TDIST_SP_DECODE_NVLS", "1") == "1"


def create_sp_decode_context(rank: int, world: int, max_batch: int, Hq: int, head_dim: int, heap=None, group=None,
                             device=None, device_epoch: bool = False) -> SpDecodeContext:
    ctx = SpDecodeContext(rank, world, max_batch, Hq, head_dim, group=group)
    on_cuda = (device is not None and torch.device(device).type == "cuda") or (device is None and torch.cuda.is_available())
    if on_cuda:
        heap = heap or symm_heap(group)
        half = world * max_batch * Hq * (head_dim + 2) // 2 * 16
        ctx.gather = heap.zeros((2, half), torch.uint8)
        if device_epoch:
            ctx.epoch_dev = torch.zeros(2, dtype=torch.int32, device=ctx.gather.local.device)
    return ctx


@nvtx_range("tdist.sp_gqa_fwd_batch_decode")
def sp_gqa_fwd_batch_decode(ctx: SpDecodeContext, q, k_cache, v_cache, global_kv_lens, block_table, scale=None,
                            soft_cap: float = 0.0, kv_split: int = -1, out: Optional[torch.Tensor] = None,
                            phase: int = 3):
    """Sequence-parallel decode step: every rank holds a contiguous shard of each sequence's KV in
    its own paged cache (``global_kv_lens[r, b]`` keys on rank r), q is replicated; returns the
    attention over the whole sequence, ``[B, Hq, D]``, identical on every rank. One launch."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    B, Hq, D = q.shape
    if q.device.type != "cuda":
        o, lse = ref_paged_attn(q, k_cache, v_cache, global_kv_lens[ctx.rank], block_table, scale, soft_cap, return_lse=True)
        mine = torch.cat([o, lse.unsqueeze(-1)], dim=-1)
        if ctx.world > 1:
            parts = [torch.empty_like(mine) for _ in range(ctx.world)]
            dist.all_gather(parts, mine, group=ctx.group)
            mine = torch.stack(parts)
        else:
            mine = mine.unsqueeze(0)
        return ref_lse_merge(mine).to(q.dtype)
    if B > ctx.max_batch or Hq != ctx.Hq or D != ctx.head_dim:
        raise ValueError("shape exceeds the sequence-parallel context")
    o = out if out is not None else torch.empty_like(q)
    # with a heap bound to an NVSwitch multicast object (TDIST_NVLS=1) the exchange stores every packet once
    mc = ctx.gather.mc if (ctx.gather.mc is not None and ctx.world > 1 and SP_DECODE_NVLS) else None
    if ctx.epoch_dev is not None:
        halves = ctx.gather.half_ptr_arrays()
        return _launch(q, k_cache, v_cache, global_kv_lens[ctx.rank], block_table, scale, soft_cap, o, 2, kv_split,
                       max_kv=int(block_table.shape[1]) * k_cache.shape[1], ll_ptrs=halves[0], ll_ptrs_odd=halves[1],
                       world=ctx.world, rank=ctx.rank, epoch=0, push_only=(phase == 1), epoch_dev=ctx.epoch_dev,
                       ll_mc=None if mc is None else mc[0].data_ptr(), ll_mc_odd=None if mc is None else mc[1].data_ptr())
    if phase != 2:
        ctx.epoch += 1  # phase 1 = compute and send only, phase 2 = redo with the same epoch and gather
    half = ctx.epoch & 1
    # the kernel strides the per-source slots by B*Hq*(D+2)/2 packets: every rank passes the same B
    # (q is replicated)
    return _launch(q, k_cache, v_cache, global_kv_lens[ctx.rank], block_table, scale, soft_cap, o, 2, kv_split,
                   max_kv=int(block_table.shape[1]) * k_cache.shape[1],
                   ll_ptrs=ctx.gather.half_ptr_arrays()[half], world=ctx.world, rank=ctx.rank, epoch=ctx.epoch,
                   push_only=(phase == 1), ll_mc=None if mc is None else mc[half].data_ptr())


kernel_inter_rank_gqa_fwd_batch_decode_combine_kv = inter_rank_combine   # the reference's name of the cross-rank merge
