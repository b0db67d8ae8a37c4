"""Tensor-parallel MoE ops on one GPU (ranks emulated send-half / receive-half). Oracle: masked
per-expert fp32 matmuls, as in the reference's test_ag_moe.py:24-39 and test_moe_reduce_rs.py."""
import pytest
import torch

from triton_distributed_b200.ops import moe_tp as MT
from triton_distributed_b200.ops import moe_utils as MU
from triton_distributed_b200.runtime import LocalWorld, check_status

pytestmark = pytest.mark.gpu


def _expert_matmul(rows, ids, b_ekn):
    out = torch.zeros(rows.shape[0], b_ekn.shape[2], device=rows.device)
    for e in range(b_ekn.shape[0]):
        m = ids == e
        if m.any():
            out[m] = rows[m].float() @ b_ekn[e].float()
    return out


@pytest.mark.parametrize("T,E,K,N,topk", [(256, 8, 256, 512, 2), (1000, 32, 520, 264, 4), (64, 60, 128, 1024, 6)])
def test_group_gemm_blocks_pick_their_expert(cuda_device, T, E, K, N, topk):
    torch.manual_seed(T + E)
    x = torch.randn(T, K, device=cuda_device).to(torch.bfloat16)
    b = (torch.randn(E, K, N, device=cuda_device) * K ** -0.5).to(torch.bfloat16)
    ids = torch.randint(0, E, (T, topk), dtype=torch.int32, device=cuda_device)
    sorted_ids, expert_ids, _, _, post_pad = MU.sort_topk_ids_align_block_size(ids, E, 1, T, 128)
    n = int(post_pad)
    a_sorted, pos_of = MT.gather_rows(x, sorted_ids[:n].contiguous(), topk, T * topk, want_inverse=True)
    c = MT.group_gemm(a_sorted, b.transpose(1, 2).contiguous(), expert_ids, (post_pad // 128).to(torch.int32))
    check_status()
    got = c[pos_of.long()].float()
    ref = _expert_matmul(x[torch.arange(T * topk, device=cuda_device) // topk], ids.reshape(-1), b)
    torch.testing.assert_close(got, ref, atol=3e-2, rtol=3e-2)
    red = MT.topk_reduce(c, pos_of, torch.ones(T, topk, device=cuda_device), T, topk)
    torch.testing.assert_close(red.float(), ref.view(T, topk, N).sum(1), atol=6e-2, rtol=3e-2)


@pytest.mark.parametrize("world,tpr,E,K,N,topk", [(1, 256, 8, 256, 256, 2), (4, 128, 16, 512, 264, 2), (8, 64, 32, 256, 512, 4)])
@pytest.mark.parametrize("mode", ["fused", "cp_async", "staged"])
def test_ag_group_gemm(cuda_device, monkeypatch, world, tpr, E, K, N, topk, mode):
    """`fused`: the all-gather only sends; one grouped-GEMM launch stages the rows block by block as the source
    rank's segment arrives, feeds the MMAs by TMA from this rank's own blocks on, and stores every row at its
    (token, k) position. `cp_async`: the producer warps gather by index. `staged`: four separate launches."""
    monkeypatch.setattr(MT, "AG_GROUP_GEMM_MODE", mode)
    torch.manual_seed(world * 7 + tpr)
    lw = LocalWorld(world, cuda_device)
    M = world * tpr
    shards = [torch.randn(tpr, K, device=cuda_device).to(torch.bfloat16) for _ in range(world)]
    bs = [(torch.randn(E, K, N, device=cuda_device) * K ** -0.5).to(torch.bfloat16) for _ in range(world)]
    ids = torch.randint(0, E, (M, topk), dtype=torch.int32, device=cuda_device)
    ctxs = [MT.create_ag_group_gemm_intra_node_context(None, shards[r], bs[r], ids, E, max_M=M, rank=r, num_ranks=world,
                                                       heap=lw.heap(r)) for r in range(world)]
    for it in range(2):   # two calls: both gather buffers
        if it == 1:
            shards = [torch.randn(tpr, K, device=cuda_device).to(torch.bfloat16) for _ in range(world)]
        if world > 1:
            for r in range(world):
                MT.ag_group_gemm_intra_node(shards[r], bs[r], ctxs[r], phase=1)
        outs = [MT.ag_group_gemm_intra_node(shards[r], bs[r], ctxs[r], phase=2 if world > 1 else 3) for r in range(world)]
        check_status()
        full = torch.cat(shards)
        rows = full[torch.arange(M * topk, device=cuda_device) // topk]
        for r in range(world):
            ref = _expert_matmul(rows, ids.reshape(-1), bs[r])
            torch.testing.assert_close(outs[r].float(), ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("world,M,E,Kl,N,topk", [(1, 256, 8, 256, 256, 2), (2, 512, 16, 128, 512, 2), (4, 256, 32, 256, 1024, 4)])
@pytest.mark.parametrize("fused", [True, False], ids=["fused_topk_rs", "staged"])
def test_moe_reduce_rs(cuda_device, monkeypatch, world, M, E, Kl, N, topk, fused):
    """`fused`: the rows are sorted by expert inside the grouped-GEMM launch and the top-k weighted reduce happens
    inside the reduce-scatter kernel (the [M, N] partial is never written); staged: row-gather kernel, grouped GEMM,
    top-k reduce kernel, plain reduce-scatter."""
    monkeypatch.setattr(MT, "FUSED_TOPK_RS", fused)
    monkeypatch.setattr(MT, "AG_GROUP_GEMM_MODE", "fused" if fused else "staged")
    torch.manual_seed(world * 11 + M)
    lw = LocalWorld(world, cuda_device)
    ids = torch.randint(0, E, (M, topk), dtype=torch.int32, device=cuda_device)
    w = torch.rand(M, topk, device=cuda_device)
    a = [torch.randn(M * topk, Kl, device=cuda_device).to(torch.bfloat16) for _ in range(world)]
    b = [(torch.randn(E, Kl, N, device=cuda_device) * (Kl * world) ** -0.5).to(torch.bfloat16) for _ in range(world)]
    ctxs = [MT.create_moe_rs_context(None, r, world, world, M, N, E, topk, torch.bfloat16, torch.bfloat16, cuda_device,
                                     full_topk_ids=ids, full_topk_weight=w, heap=lw.heap(r)) for r in range(world)]
    for it in range(2):   # two calls: both staging parities
        if it == 1:
            a = [torch.randn(M * topk, Kl, device=cuda_device).to(torch.bfloat16) for _ in range(world)]
        for r in range(world):
            MT.moe_reduce_rs(r, world, world, a[r], b[r], ctxs[r], phase=1)
        outs = [MT.moe_reduce_rs(r, world, world, a[r], b[r], ctxs[r], phase=2) for r in range(world)]
        check_status()
        total = sum((_expert_matmul(a[r], ids.reshape(-1), b[r]).view(M, topk, N) * w.view(M, topk, 1)).sum(1) for r in range(world))
        mpr = M // world
        for r in range(world):
            torch.testing.assert_close(outs[r].float(), total[r * mpr:(r + 1) * mpr], atol=6e-2, rtol=3e-2)


@pytest.mark.parametrize("T,E,K,N,topk", [(300, 8, 264, 520, 2), (128, 4, 64, 256, 1), (777, 16, 1024, 384, 3)])
def test_group_gemm_gathers_rows_in_kernel(cuda_device, T, E, K, N, topk):
    """The cp.async row-gathering producer against the staged path (row gather kernel + TMA-fed grouped GEMM):
    same sorted layout, ragged K (not a multiple of the 64-wide K block), padding rows."""
    torch.manual_seed(T + K)
    x = torch.randn(T, K, device=cuda_device).to(torch.bfloat16)
    b = (torch.randn(E, N, K, device=cuda_device) * K ** -0.5).to(torch.bfloat16)
    ids = torch.randint(0, E, (T, topk), dtype=torch.int32, device=cuda_device)
    sorted_ids, expert_ids, _, _, post_pad = MU.sort_topk_ids_align_block_size(ids, E, 1, T, 128)
    n = int(post_pad)
    sid = sorted_ids[:n].contiguous()
    nb = (post_pad // 128).to(torch.int32)
    a_sorted, _ = MT.gather_rows(x, sid, topk, T * topk)
    want = MT.group_gemm(a_sorted, b, expert_ids, nb)
    row_index = torch.div(sid, topk, rounding_mode="floor").to(torch.int32)
    got = MT.group_gemm_gather(x, row_index, b, expert_ids, nb)
    check_status()
    assert torch.equal(got, want)


@pytest.mark.parametrize("T,E,K,N,topk,rot", [(300, 8, 264, 520, 2, 0), (1500, 16, 512, 776, 3, 7), (128, 4, 64, 256, 1, 1)])
def test_group_gemm_staged_gather_rotation_and_scatter(cuda_device, T, E, K, N, topk, rot):
    """In-launch row staging (all-thread prologue + epilogue warps) + TMA-fed MMAs + scattering epilogue in one launch against the four-launch path, over several
    calls with fresh data (the per-block flags carry the call number), starting the schedule at block `rot`."""
    torch.manual_seed(T + K)
    b = (torch.randn(E, N, K, device=cuda_device) * K ** -0.5).to(torch.bfloat16)
    ids = torch.randint(0, E, (T, topk), dtype=torch.int32, device=cuda_device)
    sorted_ids, expert_ids, _, _, post_pad = MU.sort_topk_ids_align_block_size(ids, E, 1, T, 128)
    n = int(post_pad)
    sid = sorted_ids[:n].contiguous()
    nb = (post_pad // 128).to(torch.int32)
    row_index = torch.div(sid, topk, rounding_mode="floor").to(torch.int32)
    staging = torch.full((n, K), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    ready = MT.staging_flags(n, cuda_device)
    rot_t = torch.tensor([min(rot, n // 128 - 1)], dtype=torch.int32, device=cuda_device)
    for call in range(1, 4):
        x = torch.randn(T, K, device=cuda_device).to(torch.bfloat16)
        a_sorted, pos_of = MT.gather_rows(x, sid, topk, T * topk, want_inverse=True)
        want_sorted = MT.group_gemm(a_sorted, b, expert_ids, nb)
        want, _ = MT.gather_rows(want_sorted, pos_of, 1, n)
        got_sorted = MT.group_gemm_gather(x, row_index, b, expert_ids, nb, staging=staging, block_ready=ready, epoch=2 * call - 1,
                                          block_rot=rot_t)
        staging.fill_(float("nan"))    # the second launch must stage the rows again, not reuse what is there
        got = MT.group_gemm_gather(x, row_index, b, expert_ids, nb, staging=staging, block_ready=ready, epoch=2 * call,
                                   block_rot=rot_t, c_scatter=sid, c_rows=T * topk)
        check_status()
        live = sid < T * topk
        assert torch.equal(got_sorted[live], want_sorted[live])
        assert torch.equal(got, want)
        assert int(ready[n // 128:].abs().sum()) == 0      # the kernel leaves its counters at zero for the next launch
