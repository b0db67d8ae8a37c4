"""`torch.ops.tdist.*` registrations: every op is reachable through the dispatcher, runs on CPU
tensors (the torch restatement path) and has a fake implementation that yields the right shapes."""

import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import triton_distributed_b200.torch_ops as T
from triton_distributed_b200.ops import gemm as G


def test_every_op_is_registered():
    for name in T.OP_NAMES:
        assert hasattr(torch.ops.tdist, name), name


def test_gemm_family_through_the_dispatcher_on_cpu():
    torch.manual_seed(0)
    a, b = torch.randn(16, 32), torch.randn(24, 32)
    torch.testing.assert_close(torch.ops.tdist.gemm(a, b), a @ b.t())
    h = T.register_context(G.create_ag_gemm_intra_node_context(a, b, 0, 1, max_M=16))
    torch.testing.assert_close(torch.ops.tdist.ag_gemm(a, b, h), a @ b.t())
    h2 = T.register_context(G.create_gemm_rs_context(16, 24, 0, 1, device="cpu"))
    torch.testing.assert_close(torch.ops.tdist.gemm_rs(a, b, h2), a @ b.t())
    T.release_context(h)
    T.release_context(h2)


def test_decode_and_moe_ops_on_cpu():
    torch.manual_seed(1)
    q = torch.randn(2, 8, 64)
    k, v = torch.randn(6, 4, 2, 64), torch.randn(6, 4, 2, 64)
    table = torch.arange(6, dtype=torch.int32).view(2, 3)
    lens = torch.tensor([5, 12], dtype=torch.int32)
    out = torch.ops.tdist.gqa_fwd_batch_decode(q, k, v, lens, table, 0.125, 0.0)
    part = torch.ops.tdist.gqa_fwd_batch_decode_intra_rank(q, k, v, lens, table, 0.125, 0.0)
    torch.testing.assert_close(out, part[..., :64], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(torch.ops.tdist.lse_combine(torch.stack([part, part])).float(), out, atol=2e-2, rtol=2e-2)
    ids, w = torch.ops.tdist.moe_topk_softmax(torch.randn(5, 16), 2, True)
    assert ids.shape == (5, 2) and torch.allclose(w.sum(-1), torch.ones(5))
    outs = torch.ops.tdist.moe_ag_scatter_align_block_size(torch.randint(0, 4, (8, 2), dtype=torch.int32), 4, 2, 4, 4)
    assert len(outs) == 5 and int(outs[4]) % 4 == 0


def test_fake_implementations_propagate_shapes():
    a, b = torch.randn(16, 32), torch.randn(24, 32)
    h = T.register_context(G.create_ag_gemm_intra_node_context(a, b, 0, 4, max_M=64))
    with FakeTensorMode():
        fa, fb = torch.empty(16, 32), torch.empty(24, 32)
        assert torch.ops.tdist.gemm(fa, fb).shape == (16, 24)
        assert torch.ops.tdist.ag_gemm(fa, fb, h).shape == (64, 24)
        q = torch.empty(2, 8, 64)
        cache = torch.empty(6, 4, 2, 64)
        assert torch.ops.tdist.gqa_fwd_batch_decode_intra_rank(q, cache, cache, torch.empty(2, dtype=torch.int32),
                                                                 torch.empty(2, 3, dtype=torch.int32), 0.1, 0.0).shape == (2, 8, 65)
        ids, w = torch.ops.tdist.moe_topk_softmax(torch.empty(5, 16), 2, False)
        assert ids.shape == (5, 2) and w.dtype == torch.float32
    T.release_context(h)


def test_fp8_ops_through_the_dispatcher_on_cpu():
    from triton_distributed_b200.ops import gemm_fp8 as F8

    torch.manual_seed(2)
    x, w = torch.randn(16, 256), torch.randn(24, 256) * 256 ** -0.5
    a, sa = F8.quantize_fp8_rowwise(x)
    b, sb = F8.quantize_fp8_blockwise(w)
    ref = F8.gemm_fp8_reference(a, sa, b, sb)
    torch.testing.assert_close(torch.ops.tdist.gemm_fp8(a, sa, b, sb), ref)
    h = T.register_context(F8.create_ag_gemm_fp8_context(16, 256, 0, 1, device="cpu"))
    torch.testing.assert_close(torch.ops.tdist.ag_gemm_fp8(a, sa, b, sb, h), ref)
    assert (ref.float() - x @ w.t()).abs().max() < 0.1 * (x @ w.t()).abs().max()     # the quantisation itself is sane
    with FakeTensorMode():
        fa, fb = torch.empty(16, 256, dtype=F8.FP8), torch.empty(24, 256, dtype=F8.FP8)
        out = torch.ops.tdist.gemm_fp8(fa, torch.empty(16, 2), fb, torch.empty(1, 2))
        assert out.shape == (16, 24) and out.dtype == torch.bfloat16
    T.release_context(h)


def test_expert_parallel_ops_through_the_dispatcher_on_cpu():
    from triton_distributed_b200.ops import all_to_all as A
    from triton_distributed_b200.ops import moe_ep as EP

    torch.manual_seed(3)
    T_, H, E, K = 12, 256, 4, 2
    x = torch.randn(T_, H).to(torch.bfloat16)
    w, ids = torch.softmax(torch.randn(T_, E), -1).topk(K, dim=-1)
    # expert-major bf16 exchange, plain sum on the way back
    h = T.register_context(EP.create_ep_context(T_, H, K, E, 0, 1, compact=True, align=4, device="cpu"))
    rows, splits, num = torch.ops.tdist.ep_dispatch(x, ids.int(), h)
    assert int(num) == T_ * K and splits.shape == (1, E)
    torch.testing.assert_close(torch.ops.tdist.ep_combine(rows, h).float(), x.float() * K, atol=2e-2, rtol=2e-2)
    with FakeTensorMode():
        r, s, n = torch.ops.tdist.ep_dispatch(torch.empty(T_, H, dtype=torch.bfloat16), torch.empty(T_, K, dtype=torch.int32), h)
        assert r.shape[1] == H and s.shape == (1, E) and n.shape == (1,)
    T.release_context(h)
    # the quantising pair
    h2 = T.register_context(A.create_moe_dispatch_context(T_, H, K, E, 0, 1, device="cpu"))
    rx, rs, sp = torch.ops.tdist.moe_dispatch(x, ids.int(), w, h2)
    out = torch.ops.tdist.moe_combine(A.dequant_fp8(rx, rs), sp, h2)
    q, sc = A.quant_fp8_reference(x)
    torch.testing.assert_close(out.float(), A.dequant_fp8(q, sc).float() * w.sum(-1, keepdim=True), atol=3e-2, rtol=3e-2)
    with FakeTensorMode():
        frx, frs, fsp = torch.ops.tdist.moe_dispatch(torch.empty(T_, H, dtype=torch.bfloat16), torch.empty(T_, K, dtype=torch.int32),
                                                     torch.empty(T_, K), h2)
        assert frx.dtype == torch.float8_e4m3fn and frs.shape[1] == H // 128 and fsp.shape == (1, E)
    T.release_context(h2)
