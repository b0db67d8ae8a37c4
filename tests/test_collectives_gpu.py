"""Standalone collectives with all ranks emulated on one GPU: every rank's send half runs first,
then every rank's receive half, so no kernel ever waits for a kernel that has not run.
Exactness follows the reference's test_fast_allgather.py / test_reduce_scatter.py (byte-exact
all-gather, int32 reduce-scatter with atol 0)."""
import pytest
import torch

from triton_distributed_b200.ops import collectives as CO
from triton_distributed_b200.runtime import LocalWorld, check_status

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["pull", "push2d", "push_ordered", "push2d_ll"])
@pytest.mark.parametrize("world,seg", [(2, 4096), (4, 40), (8, 1 << 20), (4, 33 * 16 + 8)])
def test_fast_allgather_modes(cuda_device, mode, world, seg):
    torch.manual_seed(seg)
    lw = LocalWorld(world, cuda_device)
    ctxs = [CO.create_fast_allgather_context(r, 0, world, 1, max_buffer_size=world * seg, heap=lw.heap(r), device=cuda_device)
            for r in range(world)]
    bufs = [lw.heap(r).empty((world * seg,), torch.uint8) for r in range(world)]
    segs = [torch.randint(0, 256, (seg,), dtype=torch.uint8, device=cuda_device) for _ in range(world)]
    for it in range(3):  # epochs and LL parities
        for r in range(world):
            bufs[r].local.fill_(0xEE)
            segs[r] = (segs[r] + 1 + it)
            bufs[r].local[r * seg:(r + 1) * seg].copy_(segs[r])
        for r in range(world):
            CO.fast_allgather(bufs[r], ctxs[r], mode=mode, phase=1)
        for r in range(world):
            CO.fast_allgather(bufs[r], ctxs[r], mode=mode, phase=2)
        check_status()
        expect = torch.cat(segs)
        for r in range(world):
            assert torch.equal(bufs[r].local, expect), f"rank {r} iteration {it}"


@pytest.mark.parametrize("dtype", [torch.int32, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world,mpr,N", [(2, 8, 64), (4, 100, 256), (8, 128, 1024)])
def test_reduce_scatter(cuda_device, dtype, world, mpr, N):
    torch.manual_seed(world + mpr)
    lw = LocalWorld(world, cuda_device)
    M = world * mpr
    ctxs = [CO.create_reduce_scater_2d_ctx(M, N, r, world, dtype=dtype, heap=lw.heap(r), device=cuda_device) for r in range(world)]
    for it in range(3):
        if dtype == torch.int32:
            inputs = [torch.randint(-1000, 1000, (M, N), dtype=dtype, device=cuda_device) for _ in range(world)]
        else:
            inputs = [torch.randn(M, N, device=cuda_device).to(dtype) for _ in range(world)]
        outs = [torch.empty(mpr, N, dtype=dtype, device=cuda_device) for _ in range(world)]
        for r in range(world):
            CO.reduce_scatter_2d_op(inputs[r], ctxs[r], out=outs[r], phase=1)
        for r in range(world):
            CO.reduce_scatter_2d_op(inputs[r], ctxs[r], out=outs[r], phase=2)
        check_status()
        total = sum(x.to(torch.float64) for x in inputs)
        for r in range(world):
            ref = total[r * mpr:(r + 1) * mpr]
            if dtype == torch.int32:
                assert torch.equal(outs[r].to(torch.float64), ref)
            else:
                torch.testing.assert_close(outs[r].to(torch.float64), ref, atol=3e-2 if dtype == torch.bfloat16 else 1e-5, rtol=2e-2)


def test_ring_reduce(cuda_device):
    x = torch.randn(8 * 16, 32, device=cuda_device, dtype=torch.bfloat16)
    out = torch.empty(16, 32, device=cuda_device, dtype=torch.bfloat16)
    CO.ring_reduce(x, out, begin_idx=3, num_splits=8)
    torch.testing.assert_close(out.float(), x.float().view(8, 16, 32).sum(0), atol=5e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32, torch.int32])
@pytest.mark.parametrize("splits,begin", [(1, 0), (3, 2), (8, 5)])
def test_ring_reduce_copy_and_add_kernels(cuda_device, dtype, splits, begin):
    """Standalone reduce / copy / add helpers against torch in fp32 (exact for int32)."""
    from triton_distributed_b200.ops import collectives as CO
    torch.manual_seed(splits * 10 + begin)
    M, N = 96, 520
    if dtype == torch.int32:
        x = torch.randint(-1000, 1000, (splits * M, N), device=cuda_device, dtype=dtype)
    else:
        x = torch.randn(splits * M, N, device=cuda_device).to(dtype)
    out = torch.empty(M, N, device=cuda_device, dtype=dtype)
    before = CO.launch_count
    CO.ring_reduce(x, out, begin, splits)
    assert CO.launch_count == before + 1            # the CUDA kernel ran, not the torch fallback
    ref = x.view(splits, M, N).to(torch.float32 if dtype != torch.int32 else torch.int64).sum(0)
    if dtype == torch.int32:
        assert torch.equal(out.to(torch.int64), ref)
    else:
        torch.testing.assert_close(out.float(), ref, atol=2e-2 if dtype != torch.float32 else 1e-5, rtol=2e-2 if dtype != torch.float32 else 1e-5)
    y = torch.empty_like(x)
    CO.copy_continuous(x, y)
    assert torch.equal(x, y)
    if dtype != torch.int32:
        z = CO.add_continuous(x[:M], x[:M])
        torch.testing.assert_close(z.float(), 2 * x[:M].float(), atol=2e-2, rtol=2e-2)
