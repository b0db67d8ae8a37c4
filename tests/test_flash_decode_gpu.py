"""Flash decode on one GPU against a plain fp32 paged-attention statement; parameter grid follows
the reference's test_decode_attn.py:126-293 (kv_lens incl. 1, heads (16,16),(32,8),(64,8),(6,1),
D in {128,256}, atol 1e-2) and its sequence-parallel check (test_sp_decode_attn.py, atol 0.05)."""
import math

import pytest
import torch

from triton_distributed_b200.ops import flash_decode as FD
from triton_distributed_b200.runtime import LocalWorld, check_status

pytestmark = pytest.mark.gpu


def _make_cache(B, kv_lens, Hkv, D, page, dtype, dev, shuffle=True):
    max_blocks = max(1, (max(kv_lens) + page - 1) // page)
    nblocks = B * max_blocks + 3
    k = torch.randn(nblocks, page, Hkv, D, device=dev).to(dtype)
    v = torch.randn(nblocks, page, Hkv, D, device=dev).to(dtype)
    perm = torch.randperm(nblocks, device=dev) if shuffle else torch.arange(nblocks, device=dev)
    table = perm[: B * max_blocks].view(B, max_blocks).to(torch.int32)
    return k, v, table


@pytest.mark.parametrize("Hq,Hkv", [(16, 16), (32, 8), (64, 8), (6, 1), (96, 12)])
@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("kv_lens", [[1], [17, 300], [4096, 1, 1023, 2048]])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_decode_matches_reference(cuda_device, Hq, Hkv, D, kv_lens, dtype):
    torch.manual_seed(Hq * D + len(kv_lens))
    B, page = len(kv_lens), 16
    q = torch.randn(B, Hq, D, device=cuda_device).to(dtype)
    k, v, table = _make_cache(B, kv_lens, Hkv, D, page, dtype, cuda_device)
    lens = torch.tensor(kv_lens, dtype=torch.int32, device=cuda_device)
    scale = 1.0 / math.sqrt(D)
    out = FD.gqa_fwd_batch_decode(q, k, v, None, None, lens, table, scale)
    check_status()
    ref = FD.ref_paged_attn(q, k, v, lens, table, scale)
    torch.testing.assert_close(out.float(), ref, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("splits", [1, 3, 8, 16, 32])   # up to 8: one cluster per (batch, kv head), merged through shared memory
@pytest.mark.parametrize("soft_cap", [0.0, 30.0])
def test_intra_rank_partials_and_merge(cuda_device, splits, soft_cap):
    torch.manual_seed(splits)
    B, Hq, Hkv, D, page = 3, 32, 8, 128, 64
    kv_lens = [777, 0, 5000]
    q = torch.randn(B, Hq, D, device=cuda_device).to(torch.bfloat16)
    k, v, table = _make_cache(B, kv_lens, Hkv, D, page, torch.bfloat16, cuda_device)
    lens = torch.tensor(kv_lens, dtype=torch.int32, device=cuda_device)
    scale = 0.09
    part = FD.gqa_fwd_batch_decode_intra_rank(q, k, v, None, None, lens, table, scale, soft_cap, kv_split=splits)
    check_status()
    ro, rl = FD.ref_paged_attn(q, k, v, lens, table, scale, soft_cap, return_lse=True)
    torch.testing.assert_close(part[..., :D], ro, atol=1e-2, rtol=1e-2)
    torch.testing.assert_close(part[[0, 2], :, D], rl[[0, 2]], atol=2e-3, rtol=2e-3)
    assert torch.isinf(part[1, :, D]).all()
    # two "ranks" merged by the standalone combine kernel
    parts = torch.stack([part, part])
    merged = FD.inter_rank_combine(parts, torch.bfloat16)
    torch.testing.assert_close(merged.float(), ro, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("world,B", [(2, 1), (4, 3), (8, 8)])
def test_sequence_parallel_decode_emulated(cuda_device, world, B):
    """Every emulated rank computes and sends first; then every rank redoes its step and gathers."""
    torch.manual_seed(world * 10 + B)
    Hq, Hkv, D, page = 32, 8, 128, 16
    lw = LocalWorld(world, cuda_device)
    ctxs = [FD.create_sp_decode_context(r, world, B, Hq, D, heap=lw.heap(r), device=cuda_device) for r in range(world)]
    q = torch.randn(B, Hq, D, device=cuda_device).to(torch.bfloat16)
    for it in range(3):
        glens = torch.randint(0, 600, (world, B), dtype=torch.int32, device=cuda_device)
        glens[0, 0] = 5  # at least one key somewhere
        if it == 1:
            glens[1 % world] = 0  # a rank with no keys at all
        shards = [_make_cache(B, [max(1, int(x)) for x in glens[r]], Hkv, D, page, torch.bfloat16, cuda_device) for r in range(world)]
        for r in range(world):
            FD.sp_gqa_fwd_batch_decode(ctxs[r], q, shards[r][0], shards[r][1], glens, shards[r][2], phase=1)
        outs = [FD.sp_gqa_fwd_batch_decode(ctxs[r], q, shards[r][0], shards[r][1], glens, shards[r][2], phase=2) for r in range(world)]
        check_status()
        parts = []
        for r in range(world):
            o, l = FD.ref_paged_attn(q, shards[r][0], shards[r][1], glens[r], shards[r][2], 1.0 / math.sqrt(D), return_lse=True)
            parts.append(torch.cat([o, l.unsqueeze(-1)], -1))
        ref = FD.ref_lse_merge(torch.stack(parts))
        for r in range(world):
            torch.testing.assert_close(outs[r].float(), ref, atol=5e-2, rtol=5e-2)


@pytest.mark.parametrize("world,B", [(2, 2), (4, 3)])
@pytest.mark.parametrize("graph", [False, True], ids=["eager", "cuda_graph"])
def test_sequence_parallel_decode_with_device_call_number(cuda_device, world, B, graph):
    """The call number lives in device memory and the kernel advances it, so the launches of a step (all
    emulated ranks send, then all redo and gather) can be captured once and replayed: every replay uses the
    next number and the other buffer parity."""
    torch.manual_seed(world * 7 + B)
    Hq, Hkv, D, page = 32, 8, 128, 16
    lw = LocalWorld(world, cuda_device)
    ctxs = [FD.create_sp_decode_context(r, world, B, Hq, D, heap=lw.heap(r), device=cuda_device, device_epoch=True)
            for r in range(world)]
    q = torch.randn(B, Hq, D, device=cuda_device).to(torch.bfloat16)
    glens = torch.randint(1, 600, (world, B), dtype=torch.int32, device=cuda_device)
    shards = [_make_cache(B, [600] * B, Hkv, D, page, torch.bfloat16, cuda_device) for r in range(world)]
    outs = [torch.empty_like(q) for _ in range(world)]

    def step():
        for r in range(world):
            FD.sp_gqa_fwd_batch_decode(ctxs[r], q, shards[r][0], shards[r][1], glens, shards[r][2], phase=1)
        for r in range(world):
            FD.sp_gqa_fwd_batch_decode(ctxs[r], q, shards[r][0], shards[r][1], glens, shards[r][2], phase=2, out=outs[r])

    g = None
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()                       # warm-up (advances every rank's call number by one)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
    for it in range(4):
        q.copy_(torch.randn(B, Hq, D, device=cuda_device).to(torch.bfloat16))
        glens.copy_(torch.randint(1, 600, (world, B), dtype=torch.int32, device=cuda_device))
        if it == 2:
            glens[1 % world] = 0         # a rank without keys
            glens[0, :] = 9
        if g is not None:
            g.replay()
        else:
            step()
        torch.cuda.synchronize()
        check_status()
        parts = []
        for r in range(world):
            o, l = FD.ref_paged_attn(q, shards[r][0], shards[r][1], glens[r], shards[r][2], 1.0 / math.sqrt(D), return_lse=True)
            parts.append(torch.cat([o, l.unsqueeze(-1)], -1))
        ref = FD.ref_lse_merge(torch.stack(parts))
        for r in range(world):
            torch.testing.assert_close(outs[r].float(), ref, atol=5e-2, rtol=5e-2)
    done = 4 + (1 if graph else 0)
    for r in range(world):
        assert int(ctxs[r].epoch_dev[0]) == done and int(ctxs[r].epoch_dev[1]) == 0
