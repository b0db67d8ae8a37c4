"""MoE routing kernels and the low-latency all-to-all on one GPU (ranks emulated: all send halves,
then all receive halves). Oracles: torch softmax/topk/sort, the torch restatement of the aligned
sort, and a direct gather of the rows each rank should receive (the reference checks the same
against NCCL all_to_all_single, test_all_to_all.py:184-241)."""
import pytest
import torch

from triton_distributed_b200.ops import all_to_all as A
from triton_distributed_b200.ops import moe_utils as MU
from triton_distributed_b200.runtime import LocalWorld, check_status

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,E,K", [(128, 256, 8), (7, 64, 2), (1000, 32, 4), (33, 1024, 8)])
def test_topk_softmax(cuda_device, T, E, K):
    torch.manual_seed(T + E)
    logits = torch.randn(T, E, device=cuda_device)
    ids, w = MU.topk_softmax(logits, K)
    ref_ids, ref_w = MU.topk_softmax(logits.cpu(), K)
    assert torch.equal(ids.cpu(), ref_ids)
    torch.testing.assert_close(w.cpu(), ref_w, atol=1e-6, rtol=1e-4)
    _, wn = MU.topk_softmax(logits, K, renormalize=True)
    torch.testing.assert_close(wn.sum(-1).cpu(), torch.ones(T), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("T,E,K", [(128, 256, 8), (5, 16, 2), (4096, 64, 6), (600, 300, 3)])
def test_route_is_a_stable_expert_sort(cuda_device, T, E, K):
    torch.manual_seed(T)
    ids = torch.randint(0, E, (T, K), dtype=torch.int32, device=cuda_device)
    r = MU.route(ids, E)
    ref = MU.route(ids.cpu(), E)
    for got, want in zip(r, ref):
        assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("ranks,tpr,E,K,bs", [(8, 128, 32, 2, 128), (4, 1000, 8, 4, 64), (2, 17, 256, 8, 16), (1, 300, 60, 5, 128)])
def test_align_block_size_matches_oracle(cuda_device, ranks, tpr, E, K, bs):
    torch.manual_seed(ranks * tpr)
    ids = torch.randint(0, E, (ranks * tpr, K), dtype=torch.int32, device=cuda_device)
    got = MU.sort_topk_ids_align_block_size(ids, E, ranks, tpr, bs)
    want = MU.full_moe_align_block_size(ids, bs, E, ranks, tpr)
    total = int(want[4].item())
    assert int(got[4].item()) == total
    assert torch.equal(got[0], want[0])  # sorted ids incl. padding up to capacity
    nb = total // bs
    assert torch.equal(got[1][:nb], want[1][:nb]) and torch.equal(got[2][:nb], want[2][:nb])
    assert torch.equal(got[3], want[3])


def _emulated(world, fn_send, fn_recv):
    for r in range(world):
        fn_send(r)
    outs = [fn_recv(r) for r in range(world)]
    check_status()
    return outs


@pytest.mark.parametrize("world,T,E,K,H,with_scale", [(2, 16, 8, 2, 256, True), (4, 128, 32, 4, 1024, False), (8, 128, 256, 8, 7168, True)])
def test_fast_all_to_all_rows_land_in_source_slots(cuda_device, world, T, E, K, H, with_scale):
    torch.manual_seed(world + T)
    lw = LocalWorld(world, cuda_device)
    epr = E // world
    max_m = T * K
    ctxs = [A.create_all_to_all_context(max_m, H, r, E, world, epr, heap=lw.heap(r), device=cuda_device) for r in range(world)]
    for it in range(3):
        sends, cums, scales = [], [], []
        for r in range(world):
            ids = torch.randint(0, E, (T, K), dtype=torch.int32, device=cuda_device)
            rt = MU.route(ids, E)
            x = torch.randn(T, H, device=cuda_device).to(torch.bfloat16)
            sends.append(x[rt.sorted_token.long()].contiguous())
            cums.append(rt.cumsum)
            scales.append(torch.rand(T * K, device=cuda_device) if with_scale else None)
        _emulated(world, lambda r: A.fast_all_to_all(ctxs[r], sends[r], cums[r], scales[r], phase=1), lambda r: None)
        outs = [A.fast_all_to_all(ctxs[r], sends[r], cums[r], scales[r], phase=2) for r in range(world)]
        check_status()
        for d in range(world):
            splits, recv, rscale = outs[d]
            for s in range(world):
                lo, hi = int(cums[s][d * epr]), int(cums[s][(d + 1) * epr])
                assert torch.equal(recv[s * max_m: s * max_m + hi - lo], sends[s][lo:hi]), (it, d, s)
                want = cums[s][d * epr + 1:(d + 1) * epr + 1] - cums[s][d * epr:(d + 1) * epr]
                assert torch.equal(splits[s * epr:(s + 1) * epr], want)
                if with_scale:
                    assert torch.equal(rscale[s * max_m: s * max_m + hi - lo, 0], scales[s][lo:hi])
            data, _ = A.all_to_all_post_process(ctxs[d], splits, recv, rscale)
            assert data.shape[0] == int(splits.sum())


@pytest.mark.parametrize("world,T,E,K,H", [(2, 8, 4, 2, 256), (8, 128, 256, 8, 7168), (4, 100, 64, 6, 2048)])
def test_fused_dispatch_combine_roundtrip(cuda_device, world, T, E, K, H):
    """Identity experts: out[t] = sum_k w[t,k] * dequant(quant(x[t]))."""
    torch.manual_seed(world * 3 + T)
    lw = LocalWorld(world, cuda_device)
    ctxs = [A.create_moe_dispatch_context(T, H, K, E, r, world, heap=lw.heap(r), device=cuda_device) for r in range(world)]
    for it in range(2):
        xs = [torch.randn(T, H, device=cuda_device).to(torch.bfloat16) for _ in range(world)]
        routed = [MU.topk_softmax(torch.randn(T, E, device=cuda_device), K) for _ in range(world)]
        for r in range(world):
            A.moe_dispatch(ctxs[r], xs[r], routed[r][0], routed[r][1], phase=1)
        recvs = [A.moe_dispatch(ctxs[r], xs[r], routed[r][0], routed[r][1], phase=2) for r in range(world)]
        check_status()
        for r in range(world):   # per-source splits as the receiver sees them
            want = torch.stack([torch.bincount(routed[s][0].reshape(-1).long(), minlength=E)[r * (E // world):(r + 1) * (E // world)]
                                for s in range(world)])
            assert torch.equal(recvs[r][2].long(), want)
        # quantisation matches the torch statement on what rank 0 received from rank 1 (or itself)
        d, s = 0, world - 1
        rx, rs, splits = recvs[d]
        n = int(splits[s].sum())
        rt = MU.route(routed[s][0], E)
        rows = rt.sorted_token.long()[int(rt.cumsum[0]): int(rt.cumsum[E // world])]
        q_ref, s_ref = A.quant_fp8_reference(xs[s][rows])
        mm = T * K
        torch.testing.assert_close(rs[s * mm: s * mm + n], s_ref, rtol=1e-6, atol=0)
        assert (rx[s * mm: s * mm + n].view(torch.uint8).int() - q_ref.view(torch.uint8).int()).abs().max() <= 1
        # identity experts
        # identity experts: odd iterations write straight into the symmetric output buffer, even ones pass a tensor
        if it & 1:
            ys = [A.dequant_fp8(recvs[r][0], recvs[r][1], out=A.moe_expert_out_buffer(ctxs[r])) for r in range(world)]
        else:
            ys = [A.dequant_fp8(recvs[r][0], recvs[r][1]) for r in range(world)]
        outs = [None] * world
        for r in range(world):
            A.moe_combine(ctxs[r], ys[r], recvs[r][2], phase=1)
        for r in range(world):
            outs[r] = A.moe_combine(ctxs[r], ys[r], recvs[r][2], phase=2)
        check_status()
        for r in range(world):
            q, sc = A.quant_fp8_reference(xs[r])
            deq = (q.float().view(T, H // 128, 128) * sc.unsqueeze(-1)).view(T, H).to(torch.bfloat16).float()
            ref = deq * routed[r][1].sum(-1, keepdim=True)
            torch.testing.assert_close(outs[r].float(), ref, atol=2e-2, rtol=2e-2)


def test_route_rejects_out_of_range_expert_ids(cuda_device):
    """An id of -1 (a dropped pair) or E must not index shared memory: the pair is left out, its slot is -1, and the
    status block carries a bad-argument record that check_status() raises."""
    from triton_distributed_b200._lib import TdistError
    T, E, K = 64, 16, 2
    torch.manual_seed(5)
    ids = torch.randint(0, E, (T, K), dtype=torch.int32, device=cuda_device)
    ids[3, 1] = -1
    ids[40, 0] = E
    r = MU.route(ids, E)
    with pytest.raises(TdistError, match="bad argument"):
        check_status()
    ref = MU.route(ids.cpu(), E)
    assert int(r.splits.sum()) == T * K - 2
    assert torch.equal(r.splits.cpu(), ref.splits) and torch.equal(r.cumsum.cpu(), ref.cumsum)
    assert torch.equal(r.slot_of.cpu(), ref.slot_of)
    assert int(r.slot_of[3 * K + 1]) == -1 and int(r.slot_of[40 * K]) == -1
    live = T * K - 2
    assert torch.equal(r.sorted_token[:live].cpu(), ref.sorted_token[:live])
    # the aligned sort drops the same pairs: no sorted entry names them
    got = MU.sort_topk_ids_align_block_size(ids, E, 1, T, 16)
    with pytest.raises(TdistError, match="bad argument"):
        check_status()
    named = got[0][got[0] < T * K]
    assert named.numel() == live and (3 * K + 1) not in named.tolist() and (40 * K) not in named.tolist()
    # a clean call afterwards reports nothing
    MU.route(torch.randint(0, E, (T, K), dtype=torch.int32, device=cuda_device), E)
    check_status()


def test_fast_all_to_all_reports_a_destination_overflow(cuda_device):
    """More than max_m rows for one destination: max_m rows are sent, the published splits say so, and the status
    block records the bad argument instead of rows spilling into the next source's slot."""
    from triton_distributed_b200._lib import TdistError
    world, E, H, max_m = 2, 4, 256, 8
    lw = LocalWorld(world, cuda_device)
    epr = E // world
    ctxs = [A.create_all_to_all_context(max_m, H, r, E, world, epr, heap=lw.heap(r), device=cuda_device) for r in range(world)]
    # rank 0 sends 12 rows to rank 1's experts (2 and 3): 7 + 5 > max_m
    cums = torch.tensor([0, 1, 2, 9, 14], dtype=torch.int32, device=cuda_device)
    send = torch.randn(14, H, device=cuda_device).to(torch.bfloat16)
    A.fast_all_to_all(ctxs[0], send, cums, None, phase=1)
    with pytest.raises(TdistError, match="bad argument"):
        check_status()
    empty = torch.zeros(E + 1, dtype=torch.int32, device=cuda_device)   # rank 1 sends nothing
    A.fast_all_to_all(ctxs[1], send[:1], empty, None, phase=1)
    splits, recv, _ = A.fast_all_to_all(ctxs[1], send[:1], empty, None, phase=2)
    check_status()
    assert splits[:epr].tolist() == [7, 1]          # clamped to the 8 rows that were sent
    assert torch.equal(recv[:max_m], send[2:2 + max_m])


@pytest.mark.parametrize("world,T,E,K,H,align", [(2, 33, 8, 2, 256, 1), (4, 64, 32, 4, 512, 128), (8, 128, 256, 8, 1024, 128), (1, 50, 4, 3, 128, 16)])
def test_ep_dispatch_compact_layout_and_pull_combine(cuda_device, world, T, E, K, H, align):
    """Compact (expert-major) receive layout with block-aligned groups: every rank's rows sit where the gathered
    counts say, the block -> expert table covers them, and the pull combine returns K x the input (identity
    experts, plain sum). The (token, k) pairs of rank 1 include a dropped pair (id -1)."""
    from triton_distributed_b200._lib import TdistError
    from triton_distributed_b200.ops import moe_ep as EP
    torch.manual_seed(world * 11 + T)
    lw = LocalWorld(world, cuda_device)
    ctxs = [EP.create_ep_context(T, H, K, E, r, world, quant=False, compact=True, align=align, heap=lw.heap(r), device=cuda_device)
            for r in range(world)]
    epr = E // world
    for it in range(3):
        xs = [torch.randn(T, H, device=cuda_device).to(torch.bfloat16) for _ in range(world)]
        ids = [torch.randint(0, E, (T, K), dtype=torch.int32, device=cuda_device) for _ in range(world)]
        dropped = world > 1 and it == 1
        if dropped:
            ids[1][5, 0] = -1
        for phase in (1, 2):
            for r in range(world):
                EP.ep_dispatch(ctxs[r], xs[r], ids[r], None, phase=phase)
        recv = [EP.ep_dispatch(ctxs[r], xs[r], ids[r], None, phase=4) for r in range(world)]
        if dropped:
            with pytest.raises(TdistError, match="bad argument"):
                check_status()
        else:
            check_status()
        for d in range(world):
            rows, _, splits, num_recv = recv[d]
            off, total = 0, 0
            for le in range(epr):
                e = d * epr + le
                group = torch.cat([xs[s][(ids[s].reshape(-1) == e).nonzero().flatten() // K] for s in range(world)])
                n = group.shape[0]
                assert torch.equal(rows[off: off + n], group), (it, d, le)
                nb = (n + align - 1) // align
                assert (ctxs[d].block_expert[off // align: off // align + nb] == le).all()
                off += nb * align
                total += n
            assert int(num_recv) == total and int(ctxs[d].num_blocks) == off // align
        for r in range(world):
            EP.expert_out_buffer(ctxs[r]).copy_(recv[r][0])     # identity experts, written in place
            EP.ep_combine(ctxs[r], None, weighted=False, phase=1)
        outs = [EP.ep_combine(ctxs[r], None, weighted=False, phase=2) for r in range(world)]
        check_status()
        for r in range(world):
            live = (ids[r] >= 0).sum(-1, keepdim=True).float()
            torch.testing.assert_close(outs[r].float(), xs[r].float() * live, atol=2e-2, rtol=2e-2)
