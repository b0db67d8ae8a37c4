"""tcgen05 GEMM family on one GPU: plain GEMM numerics, and the fused AG / RS kernels of one
emulated rank at a time against peer buffers prepared by the host (LocalWorld).

Oracle: plain PyTorch fp32 matmul of the same operands. Mirrors the reference's
test_ag_gemm_intra_node.py / test_gemm_rs.py checks (non-tile-aligned M, stale workspace poisoning)
without needing several GPUs.
"""
import pytest
import torch

from triton_distributed_b200 import _lib
from triton_distributed_b200.ops import gemm as G
from triton_distributed_b200.runtime import LocalWorld, check_status, global_status

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1, 2], ids=["cta1", "cta_pair", "cta_pair_wide"])
def tiling(request, monkeypatch):
    """Run a test under every tiling of the kernel (one CTA per 128x256 tile, CTA pair per 256x256 tile, CTA pair
    per 256x512 tile)."""
    monkeypatch.setattr(G, "CTA_PAIR", request.param)
    return request.param


def _rand(shape, dtype, dev, scale=1.0):
    return (torch.randn(shape, device=dev, dtype=torch.float32) * scale).to(dtype)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (300, 264, 136), (1000, 1000, 992), (4096, 768, 2048),
                                   (520, 1288, 200), (8192, 1536, 1024), (2304, 5128, 320)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_plain_gemm_matches_fp32_reference(cuda_device, tiling, M, N, K, dtype):
    torch.manual_seed(M + N + K)
    a = _rand((M, K), dtype, cuda_device)
    b = _rand((N, K), dtype, cuda_device, K ** -0.5)
    c = G.gemm_persistent(a, b)
    check_status()
    ref = a.float() @ b.float().t()
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert torch.isfinite(c).all()
    torch.testing.assert_close(c.float(), ref, atol=tol, rtol=tol)


@pytest.mark.parametrize("world,mpr,N,K", [(2, 128, 256, 128), (4, 250, 520, 264), (8, 96, 256, 512), (4, 999, 768, 1024),
                                           (2, 520, 1288, 192), (4, 384, 1224, 128), (2, 130, 2048 + 64, 256)])
def test_ag_gemm_single_rank_kernels_against_prepared_peers(cuda_device, tiling, world, mpr, N, K):
    """Each emulated rank's fused kernel runs alone: blocks of lower ranks were really pushed by
    their kernels, blocks of higher ranks are written by the host together with their flags."""
    torch.manual_seed(world * 1000 + mpr)
    dtype = torch.bfloat16
    lw = LocalWorld(world, cuda_device)
    A = [_rand((mpr, K), dtype, cuda_device) for _ in range(world)]
    B = [_rand((N, K), dtype, cuda_device, K ** -0.5) for _ in range(world)]
    ctxs = [G.create_ag_gemm_intra_node_context(A[r], B[r], r, world, max_M=world * mpr + 64, heap=lw.heap(r))
            for r in range(world)]
    full = torch.cat(A).float()
    mt = (mpr + 127) // 128
    for r in range(world):
        ctx = ctxs[r]
        half = (ctx.epoch + 1) & 1
        ws = ctx.workspace.local[half][: world * mpr * K].view(world, mpr, K)
        flags = ctx.flags.local[half][: world * mt].view(world, mt)
        # poison what no kernel has written yet, then stand in for the ranks that have not run
        for s in range(r + 1, world):
            ws[s].copy_(A[s])
            flags[s].fill_(ctx.epoch + 1)
        ws[r].fill_(float("nan"))  # own slot is never read from the workspace
        c = G.ag_gemm_intra_node(A[r], B[r], ctx)
        check_status()
        ref = full @ B[r].float().t()
        torch.testing.assert_close(c.float(), ref, atol=2e-2, rtol=2e-2)
    # every rank's shard was pushed to every other rank, with its flags
    for r in range(world):
        ws = ctxs[r].workspace.local[1][: world * mpr * K].view(world, mpr, K)
        flags = ctxs[r].flags.local[1][: world * mt].view(world, mt)
        for s in range(world):
            if s == r:
                continue
            assert torch.equal(ws[s], A[s]), f"rank {r} workspace slot {s}"
            assert (flags[s] == 1).all()


@pytest.mark.parametrize("world,mpr,N,K", [(2, 128, 256, 128), (4, 250, 520, 264), (8, 96, 512, 256), (4, 512, 1024, 512),
                                           (2, 520, 1288, 192), (4, 300, 1224, 128), (2, 130, 2048 + 64, 256)])
def test_gemm_rs_single_rank_kernels_against_prepared_peers(cuda_device, tiling, world, mpr, N, K):
    torch.manual_seed(world * 77 + mpr)
    dtype = torch.bfloat16
    lw = LocalWorld(world, cuda_device)
    M = world * mpr
    A = [_rand((M, K), dtype, cuda_device) for _ in range(world)]
    B = [_rand((N, K), dtype, cuda_device, (K * world) ** -0.5) for _ in range(world)]
    partial = [(A[s].float() @ B[s].float().t()) for s in range(world)]
    total = sum(partial)
    ctxs = [G.create_gemm_rs_context(M + 8, N, r, world, heap=lw.heap(r), device=cuda_device) for r in range(world)]
    tiles = ((mpr + 127) // 128) * ((N + 255) // 256)
    for r in range(world):
        ctx = ctxs[r]
        half = (ctx.epoch + 1) & 1
        stage = ctx.staging.local[half][: world * mpr * N].view(world, mpr, N)
        flags = ctx.flags.local[half][: tiles * world].view(tiles, world)
        for s in range(r + 1, world):
            stage[s].copy_(partial[s][r * mpr:(r + 1) * mpr].to(dtype))
            flags[:, s].fill_(ctx.epoch + 1)
        out = G.gemm_rs(A[r], B[r], ctx)
        check_status()
        ref = total[r * mpr:(r + 1) * mpr]
        torch.testing.assert_close(out.float(), ref, atol=3e-2, rtol=3e-2)


def test_abandoned_wait_reports_timeout_and_leaves_the_context_usable(cuda_device, monkeypatch):
    """A flag that nothing sets: the kernel must give up after its limit, report which flag it was
    waiting for, and return, and the next launch must work."""
    monkeypatch.setenv("TDIST_WAIT_TIMEOUT_MS", "50")
    dtype = torch.bfloat16
    lw = LocalWorld(2, cuda_device)
    a = _rand((128, 128), dtype, cuda_device)
    b = _rand((256, 128), dtype, cuda_device)
    ctx = G.create_ag_gemm_intra_node_context(a, b, 0, 2, max_M=256, heap=lw.heap(0))
    G.create_ag_gemm_intra_node_context(a, b, 1, 2, max_M=256, heap=lw.heap(1))
    G.ag_gemm_intra_node(a, b, ctx)
    torch.cuda.synchronize()
    st = global_status()
    assert st.aborted()
    rec = st.record
    assert rec.code == 1 and rec.peer == 1 and rec.expected == 1
    with pytest.raises(_lib.TdistTimeoutError):
        check_status()
    # the context is still usable
    c = G.gemm_persistent(a, b)
    check_status()
    torch.testing.assert_close(c.float(), a.float() @ b.float().t(), atol=2e-2, rtol=2e-2)


def test_consumer_blocks_until_the_host_sets_the_flags(cuda_device):
    """The fused AG-GEMM of one emulated rank is launched while the peer's rows are in the workspace but their flags
    are not set; the host sets them a moment later with stream write-values (no kernel involved). The kernel must
    wait, then finish with the right result (the reference's test_distributed_wait.py `correctness` case)."""
    import time

    from triton_distributed_b200.ops import collectives as CO

    torch.manual_seed(5)
    dtype = torch.bfloat16
    world, mpr, N, K = 2, 256, 512, 256
    lw = LocalWorld(world, cuda_device)
    A = [_rand((mpr, K), dtype, cuda_device) for _ in range(world)]
    B = _rand((N, K), dtype, cuda_device, K ** -0.5)
    ctxs = [G.create_ag_gemm_intra_node_context(A[r], B, r, world, max_M=world * mpr, heap=lw.heap(r)) for r in range(world)]
    ctx = ctxs[0]
    half = (ctx.epoch + 1) & 1
    mt = (mpr + 127) // 128
    ws = ctx.workspace.local[half][: world * mpr * K].view(world, mpr, K)
    flags = ctx.flags.local[half][: world * mt].view(world, mt)
    ws[1].copy_(A[1])
    assert int(flags[1].abs().sum()) == 0          # nothing has announced rank 1's blocks
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    t0 = time.time()
    c = G.ag_gemm_intra_node(A[0], B, ctx)         # asynchronous: the kernel now spins on rank 1's flags
    time.sleep(0.3)
    for b in range(mt):
        CO.set_signal(flags[1, b:b + 1].data_ptr(), ctx.epoch, stream=side)
    torch.cuda.synchronize()
    took = time.time() - t0
    check_status()
    assert took >= 0.3                               # it really waited for the host
    ref = torch.cat(A).float() @ B.float().t()
    torch.testing.assert_close(c.float(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("N,K", [(264, 128), (320, 192), (456, 64), (1288, 128)])
def test_partial_column_tiles_over_many_fresh_inputs(cuda_device, tiling, N, K):
    """Column counts whose last 256-column tile holds 8, 64, 200 and 8 (after two and a half wide tiles) columns,
    row counts that are no multiple of 128 or 256, 20 iterations with fresh data: a stale or misplaced partial
    tile shows up as a wrong element in some iteration."""
    dtype = torch.bfloat16
    gen = torch.Generator(device=cuda_device).manual_seed(N * 7 + K)
    for it in range(20):
        M = int(torch.randint(1, 700, (1,), generator=gen, device=cuda_device))
        a = torch.randn(M, K, device=cuda_device, generator=gen).to(dtype)
        b = (torch.randn(N, K, device=cuda_device, generator=gen) * K ** -0.5).to(dtype)
        c = torch.full((M, N), float("nan"), device=cuda_device, dtype=dtype)
        G.gemm_persistent(a, b, out=c)
        check_status()
        torch.testing.assert_close(c.float(), a.float() @ b.float().t(), atol=2e-2, rtol=2e-2, msg=lambda m: f"iteration {it}, M={M}: {m}")


@pytest.mark.parametrize("world", [2, 4])
def test_gemm_rs_random_m_sweep(cuda_device, tiling, world):
    """Seeded sweep over random M (any multiple of the world size up to the context's limit), one context reused
    across the calls as in serving (the reference's test_gemm_rs.py:209-231 draws M the same way)."""
    dtype = torch.bfloat16
    N, K, max_mpr = 776, 192, 300
    gen = torch.Generator(device=cuda_device).manual_seed(world)
    lw = LocalWorld(world, cuda_device)
    ctxs = [G.create_gemm_rs_context(world * max_mpr, N, r, world, heap=lw.heap(r), device=cuda_device) for r in range(world)]
    for it in range(12):
        mpr = int(torch.randint(1, max_mpr + 1, (1,), generator=gen, device=cuda_device))
        M = world * mpr
        A = [torch.randn(M, K, device=cuda_device, generator=gen).to(dtype) for _ in range(world)]
        B = [(torch.randn(N, K, device=cuda_device, generator=gen) * (K * world) ** -0.5).to(dtype) for _ in range(world)]
        partial = [(A[s].float() @ B[s].float().t()) for s in range(world)]
        total = sum(partial)
        tiles = ((mpr + 127) // 128) * ((N + 255) // 256)
        for r in range(world):
            ctx = ctxs[r]
            half = (ctx.epoch + 1) & 1
            stage = ctx.staging.local[half][: world * mpr * N].view(world, mpr, N)
            flags = ctx.flags.local[half][: tiles * world].view(tiles, world)
            for s in range(r + 1, world):
                stage[s].copy_(partial[s][r * mpr:(r + 1) * mpr].to(dtype))
                flags[:, s].fill_(ctx.epoch + 1)
            out = G.gemm_rs(A[r], B[r], ctx)
            check_status()
            torch.testing.assert_close(out.float(), total[r * mpr:(r + 1) * mpr], atol=3e-2, rtol=3e-2,
                                       msg=lambda m: f"iteration {it}, mpr={mpr}, rank {r}: {m}")
