"""Block-scaled fp8 GEMM on one GPU: plain numerics, and the fused AG kernel of one emulated rank at a
time against peer buffers prepared by the host (LocalWorld).

Oracle: fp32 torch matmul of the dequantised operands (values = fp8 * scale), i.e. the same op
restated without tensor cores. The kernel accumulates each 128-wide K block in fp32 on the tensor
core and folds it in with an fp32 FMA, so the only rounding besides summation order is the final
bf16 store.
"""
import pytest
import torch

from triton_distributed_b200.ops import gemm_fp8 as F
from triton_distributed_b200.runtime import LocalWorld, check_status

pytestmark = pytest.mark.gpu



def _operands(M, N, K, dev, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    # per-block magnitudes spread over several octaves so that a wrong or misplaced scale is visible
    x = torch.randn(M, K, generator=g) * torch.exp2(torch.randint(-3, 4, (M, K // 128), generator=g).float()).repeat_interleave(128, 1)
    w = torch.randn(N, K, generator=g) * K ** -0.5
    wblk = torch.exp2(torch.randint(-2, 3, ((N + 127) // 128, K // 128), generator=g).float())
    w = w * wblk.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)
    a, sa = F.quantize_fp8_rowwise(x.to(dev))
    b, sb = F.quantize_fp8_blockwise(w.to(dev))
    return a, sa, b, sb


def test_quantisers_round_trip(cuda_device):
    a, sa, b, sb = _operands(200, 264, 384, cuda_device, 1)
    assert a.dtype == F.FP8 and sa.shape == (200, 3) and sb.shape == (3, 3)
    x = F.dequantize_fp8(a, sa, 1)
    a2, sa2 = F.quantize_fp8_rowwise(x)
    torch.testing.assert_close(F.dequantize_fp8(a2, sa2, 1), x, rtol=0.07, atol=1e-6)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 512), (300, 264, 384), (1000, 1000, 896), (4096, 768, 2048)])
def test_plain_fp8_gemm_matches_fp32_reference(cuda_device, M, N, K):
    a, sa, b, sb = _operands(M, N, K, cuda_device, M + N + K)
    c = F.gemm_fp8_blockscaled(a, sa, b, sb)
    check_status()
    ref = F.dequantize_fp8(a, sa, 1) @ F.dequantize_fp8(b, sb, 128).t()
    assert torch.isfinite(c).all()
    torch.testing.assert_close(c.float(), ref, atol=2e-2 * ref.abs().max().item() / 4, rtol=1e-2)


def test_fp8_gemm_is_deterministic_across_calls(cuda_device):
    a, sa, b, sb = _operands(512, 512, 1024, cuda_device, 7)
    c1 = F.gemm_fp8_blockscaled(a, sa, b, sb)
    c2 = F.gemm_fp8_blockscaled(a, sa, b, sb, num_sms=37)
    check_status()
    assert torch.equal(c1, c2)


@pytest.mark.parametrize("world,mpr,N,K", [(1, 200, 256, 256), (2, 128, 256, 128), (4, 250, 520, 384), (8, 96, 256, 512)])
def test_ag_fp8_gemm_single_rank_kernels_against_prepared_peers(cuda_device, world, mpr, N, K):
    """Each emulated rank's fused kernel runs alone: rows and scales of lower ranks were really pushed
    by their kernels, those of higher ranks are written by the host together with their flags."""
    lw = LocalWorld(world, cuda_device)
    ops = [_operands(mpr, N, K, cuda_device, 100 * world + r) for r in range(world)]
    ctxs = [F.create_ag_gemm_fp8_context(world * mpr + 64, K, r, world, device=cuda_device, heap=lw.heap(r)) for r in range(world)]
    full = torch.cat([F.dequantize_fp8(o[0], o[1], 1) for o in ops])
    mt, kb = (mpr + 127) // 128, K // 128
    for r in range(world):
        ctx = ctxs[r]
        a, sa, b, sb = ops[r]
        if world > 1:
            half = (ctx.epoch + 1) & 1
            ws = ctx.workspace.local[half][: world * mpr * K].view(world, mpr, K)
            sws = ctx.scale_ws.local[half][: world * mpr * kb].view(world, mpr, kb)
            flags = ctx.flags.local[half][: world * mt].view(world, mt)
            for s in range(r + 1, world):
                ws[s].copy_(ops[s][0].view(torch.uint8))
                sws[s].copy_(ops[s][1])
                flags[s].fill_(ctx.epoch + 1)
            ws[r].fill_(0x7F)          # e4m3 NaN: the own slot is never read from the workspace
            sws[r].fill_(float("nan"))
        c = F.ag_gemm_fp8(a, sa, b, sb, ctx)
        check_status()
        ref = full @ F.dequantize_fp8(b, sb, 128).t()
        assert torch.isfinite(c).all()
        torch.testing.assert_close(c.float(), ref, atol=2e-2 * ref.abs().max().item() / 4, rtol=1e-2)
    for r in range(world):
        if world == 1:
            break
        ws = ctxs[r].workspace.local[1][: world * mpr * K].view(world, mpr, K)
        sws = ctxs[r].scale_ws.local[1][: world * mpr * kb].view(world, mpr, kb)
        for s in range(world):
            if s != r:
                assert torch.equal(ws[s], ops[s][0].view(torch.uint8)), f"rank {r} rows of {s}"
                assert torch.equal(sws[s], ops[s][1]), f"rank {r} scales of {s}"
