"""Layer wrappers and model blocks on one GPU (world 1, or ranks emulated send-half / receive-half)."""
import math

import pytest
import torch
import torch.nn.functional as F

from triton_distributed_b200.models import AllGatherLayer, EPAll2AllLayer, EPMoE, SpGQAFlashDecodeAttention, TPMLP
from triton_distributed_b200.ops import all_to_all as A
from triton_distributed_b200.ops import flash_decode as FD
from triton_distributed_b200.runtime import LocalWorld, check_status

pytestmark = pytest.mark.gpu


def test_tp_mlp_single_rank(cuda_device):
    torch.manual_seed(0)
    M, H, Fd = 512, 1024, 2048
    x = torch.randn(M, H, device=cuda_device).to(torch.bfloat16)
    w1 = (torch.randn(Fd, H, device=cuda_device) * H ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(H, Fd, device=cuda_device) * Fd ** -0.5).to(torch.bfloat16)
    mlp = TPMLP(w1, w2, 0, 1, max_M=M)
    y = mlp(x)
    check_status()
    h = F.gelu((x.float() @ w1.float().t()).to(torch.bfloat16), approximate="tanh")
    ref = h.float() @ w2.float().t()
    torch.testing.assert_close(y.float(), ref, atol=5e-2, rtol=5e-2)


def test_ep_moe_single_rank(cuda_device):
    torch.manual_seed(1)
    T, H, Fd, E, K = 128, 512, 256, 8, 2
    x = torch.randn(T, H, device=cuda_device).to(torch.bfloat16)
    gate = torch.randn(E, H, device=cuda_device).to(torch.bfloat16)
    w1 = (torch.randn(E, Fd, H, device=cuda_device) * H ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(E, H, Fd, device=cuda_device) * Fd ** -0.5).to(torch.bfloat16)
    moe = EPMoE(gate, w1, w2, K, 0, 1, max_tokens=T)
    y = moe(x)
    check_status()
    from triton_distributed_b200.ops import moe_utils as MU
    ids, w = MU.topk_softmax(x.float() @ gate.float().t(), K, renormalize=True)
    xd = x.float()          # rows travel as bf16
    ref = torch.zeros(T, H, device=cuda_device)
    for t in range(T):
        for k in range(K):
            e = int(ids[t, k])
            h = F.silu((xd[t] @ w1[e].float().t()).to(torch.bfloat16)).float()
            ref[t] += w[t, k] * (h @ w2[e].float().t()).to(torch.bfloat16).float()
    torch.testing.assert_close(y.float(), ref, atol=6e-2, rtol=6e-2)


@pytest.mark.parametrize("world", [2, 4])
def test_ep_all2all_layer_emulated(cuda_device, world):
    torch.manual_seed(world)
    T, H, K, E = 64, 256, 4, 8 * world
    lw = LocalWorld(world, cuda_device)
    layers = [EPAll2AllLayer(None, T, H, K, r, E, world, world, heap=lw.heap(r), device=cuda_device) for r in range(world)]
    xs = [torch.randn(T, H, device=cuda_device).to(torch.bfloat16) for _ in range(world)]
    ids = [torch.randint(0, E, (T, K), dtype=torch.int32, device=cuda_device) for _ in range(world)]
    for phase in (1, 2):        # every rank publishes its counts, then every rank sends
        for r in range(world):
            layers[r].dispatch(xs[r], ids[r], phase=phase)
    recv = [layers[r].dispatch(xs[r], ids[r], phase=4) for r in range(world)]
    check_status()
    epr = E // world
    for d in range(world):
        # rows grouped by local expert then source rank, each group in the source's token order
        want = []
        for e in range(d * epr, (d + 1) * epr):
            for s in range(world):
                pairs = (ids[s].reshape(-1) == e).nonzero().flatten()
                want.append(xs[s][pairs // K])
        want = torch.cat(want)
        assert int(layers[d].num_recv) == want.shape[0]
        assert torch.equal(recv[d][: want.shape[0]], want)
        # the group table matches: splits [source, expert] and the start row of every (expert, source) group
        sp = torch.stack([torch.bincount(ids[s].reshape(-1).long(), minlength=E)[d * epr:(d + 1) * epr] for s in range(world)])
        assert torch.equal(layers[d].recv_splits.long(), sp)
        flat = sp.t().reshape(-1)
        assert torch.equal(layers[d].recv_offset.long().reshape(-1), torch.cumsum(flat, 0) - flat)
    for r in range(world):
        layers[r].combine(recv[r], phase=1)
    outs = [layers[r].combine(recv[r], phase=2) for r in range(world)]
    check_status()
    for r in range(world):
        torch.testing.assert_close(outs[r].float(), xs[r].float() * K, atol=2e-2, rtol=2e-2)


def test_allgather_layer_emulated(cuda_device):
    world = 4
    lw = LocalWorld(world, cuda_device)
    layers = [AllGatherLayer(1, world, r, max_buffer_size=1 << 20, stages=2, heap=lw.heap(r), device=cuda_device) for r in range(world)]
    for mode in ("forward_pull", "forward_push_2d", "forward_push_2d_ll"):
        segs = [torch.randn(33, 65, device=cuda_device) for _ in range(world)]
        for r in range(world):
            getattr(layers[r], mode)(segs[r], phase=1)
        outs = [getattr(layers[r], mode)(segs[r], phase=2) for r in range(world)]
        check_status()
        for r in range(world):
            assert torch.equal(outs[r], torch.stack(segs))


def test_sp_decode_layer_world1(cuda_device):
    B, Hq, Hkv, D, page = 2, 32, 8, 128, 16
    layer = SpGQAFlashDecodeAttention(0, 0, 1, 1, Hq, Hkv, D, D, page, 1.0 / math.sqrt(D), 0.0, max_allowed_batch=B, device=cuda_device)
    q = torch.randn(B, Hq, D, device=cuda_device).to(torch.bfloat16)
    k = torch.randn(64, page, Hkv, D, device=cuda_device).to(torch.bfloat16)
    v = torch.randn(64, page, Hkv, D, device=cuda_device).to(torch.bfloat16)
    table = torch.arange(64, device=cuda_device, dtype=torch.int32).view(B, 32)
    lens = torch.tensor([[500, 37]], dtype=torch.int32, device=cuda_device)
    out = layer(q, k, v, lens, table)
    check_status()
    ref = FD.ref_paged_attn(q, k, v, lens[0], table, 1.0 / math.sqrt(D))
    torch.testing.assert_close(out.float(), ref, atol=1e-2, rtol=1e-2)
