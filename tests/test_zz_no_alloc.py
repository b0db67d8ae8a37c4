"""Allocation-free flash decode (`tdist_flash_decode_static`, declared in csrc/include/tdist_noalloc.h).

Some users of the library cannot allocate device memory around a decode step: a serving loop that
must not pay for (or be stalled by) cudaMalloc / cudaFree, a host program that already handed the
whole GPU to its own memory pool, or a plain-C / ctypes caller that only has raw device pointers
and no allocator for a workspace. For them the library carries the decode kernel's scratch
(split-merge workspace + arrival counters) inside its own image, in a fixed 8 MiB device array.

The test drives the entry point the way such a caller would — through the exported C symbol, with
raw pointers — twice in a row with different problems (the array keeps the previous call's
contents, so a stale-scratch bug would show on the second call), and compares against the regular
entry point, which takes its scratch from the caller. It also checks that a problem too large for
the built-in array is refused with a clear message instead of being launched.

This file sorts last on purpose: a run that stops at the first failure has then already executed
every other test.
"""
import ctypes as C
import math

import pytest
import torch

from triton_distributed_b200 import _lib
from triton_distributed_b200.ops import flash_decode as FD
from triton_distributed_b200.runtime import check_status, default_timeout_ns, global_status

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 8 << 20


def _args(q, k, v, lens, table, out, splits, mode, scale):
    a = _lib.DecodeArgs()
    B, Hq, D = q.shape
    _, page, Hkv, _ = k.shape
    a.q, a.k_cache, a.v_cache = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.block_table, a.kv_lens, a.out = table.data_ptr(), lens.data_ptr(), out.data_ptr()
    a.B, a.Hq, a.Hkv, a.head_dim, a.page_size = B, Hq, Hkv, D, page
    a.max_blocks, a.splits = table.shape[1], splits
    a.stride_block, a.stride_token, a.stride_head = k.stride(0), k.stride(1), k.stride(2)
    a.scale, a.soft_cap, a.mode = scale, 0.0, mode
    a.dtype = _lib.DT_BF16 if q.dtype == torch.bfloat16 else _lib.DT_F16
    a.world, a.rank = 1, 0
    a.status = global_status().device_ptr
    a.timeout_ns = default_timeout_ns()
    a.stream = torch.cuda.current_stream(q.device).cuda_stream
    return a


def _problem(B, Hq, Hkv, D, kv_lens, page, dtype, dev):
    max_blocks = (max(kv_lens) + page - 1) // page
    k = torch.randn(B * max_blocks, page, Hkv, D, device=dev).to(dtype)
    v = torch.randn(B * max_blocks, page, Hkv, D, device=dev).to(dtype)
    table = torch.randperm(B * max_blocks, device=dev).view(B, max_blocks).to(torch.int32)
    q = torch.randn(B, Hq, D, device=dev).to(dtype)
    lens = torch.tensor(kv_lens, dtype=torch.int32, device=dev)
    return q, k, v, lens, table


def test_static_scratch_entry_point_matches_the_regular_one_twice(cuda_device):
    fn = _lib.lib().tdist_flash_decode_static  # the exported C symbol
    fn.argtypes = [C.POINTER(_lib.DecodeArgs)]
    fn.restype = C.c_int
    torch.manual_seed(123)
    problems = [
        dict(B=4, Hq=32, Hkv=8, D=128, kv_lens=[3000, 1, 777, 4096], page=16, dtype=torch.bfloat16, splits=9),
        dict(B=2, Hq=16, Hkv=16, D=64, kv_lens=[129, 2050], page=32, dtype=torch.float16, splits=3),
    ]
    for cfg in problems:
        splits = cfg.pop("splits")
        q, k, v, lens, table = _problem(dev=cuda_device, **cfg)
        scale = 1.0 / math.sqrt(q.shape[-1])
        expect = FD.gqa_fwd_batch_decode(q, k, v, None, None, lens, table, scale, kv_split=splits)
        got = torch.full_like(q, float("nan"))
        rc = fn(C.byref(_args(q, k, v, lens, table, got, splits, 0, scale)))
        assert rc == 0, _lib.lib().tdist_last_error()
        check_status()
        torch.testing.assert_close(got.float(), expect.float(), atol=1e-2, rtol=1e-2)
        # and against the plain PyTorch fp32 statement of paged attention, not only against the other entry point
        torch.testing.assert_close(got.float(), FD.ref_paged_attn(q, k, v, lens, table, scale), atol=2e-2, rtol=2e-2)
        # and the O || LSE form
        expect1 = FD.gqa_fwd_batch_decode_intra_rank(q, k, v, None, None, lens, table, scale, kv_split=splits)
        got1 = torch.full_like(expect1, float("nan"))
        rc = fn(C.byref(_args(q, k, v, lens, table, got1, splits, 1, scale)))
        assert rc == 0, _lib.lib().tdist_last_error()
        check_status()
        torch.testing.assert_close(got1, expect1, atol=1e-2, rtol=1e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit(cuda_device):
    fn = _lib.lib().tdist_flash_decode_static
    fn.argtypes = [C.POINTER(_lib.DecodeArgs)]
    fn.restype = C.c_int
    q, k, v, lens, table = _problem(8, 64, 8, 128, [64] * 8, 16, torch.bfloat16, cuda_device)
    out = torch.zeros_like(q)
    splits = 64  # 8*64*64*130*4 bytes = 17 MB > 8 MiB
    assert 8 * 64 * splits * 130 * 4 > STATIC_SCRATCH_BYTES
    rc = fn(C.byref(_args(q, k, v, lens, table, out, splits, 0, 0.1)))
    assert rc == -3
    msg = _lib.lib().tdist_last_error().decode()
    assert "exceeds the built-in scratch" in msg
    torch.cuda.synchronize()
    assert out.abs().sum().item() == 0  # nothing ran
