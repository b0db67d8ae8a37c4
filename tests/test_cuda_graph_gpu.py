"""Single-GPU ops inside a CUDA graph: a decode step (attention + a tcgen05 GEMM on its output + top-k routing)
is captured once and replayed with new contents in the same buffers. The launchers take the stream from
torch, allocate nothing during capture once warmed up, and read lengths and routing on the device, so the
graph stays valid when the data changes. (Ops whose flags carry a host-side call number - the fused
collectives - are not captured: every launch needs a new number.)"""
import math

import pytest
import torch

from triton_distributed_b200.ops import flash_decode as FD
from triton_distributed_b200.ops import gemm as G
from triton_distributed_b200.ops import moe_utils as MU
from triton_distributed_b200.runtime import check_status

pytestmark = pytest.mark.gpu


def test_decode_step_replays_from_a_cuda_graph(cuda_device):
    torch.manual_seed(0)
    dev = cuda_device
    B, Hq, Hkv, D, page, max_len = 4, 32, 8, 128, 16, 2048
    blocks = B * (max_len // page)
    k = torch.randn(blocks, page, Hkv, D, device=dev).to(torch.bfloat16)
    v = torch.randn(blocks, page, Hkv, D, device=dev).to(torch.bfloat16)
    table = torch.randperm(blocks, device=dev).view(B, max_len // page).to(torch.int32)
    q = torch.randn(B, Hq, D, device=dev).to(torch.bfloat16)
    lens = torch.tensor([5, 700, 2048, 1], dtype=torch.int32, device=dev)
    w_o = (torch.randn(512, Hq * D, device=dev) * (Hq * D) ** -0.5).to(torch.bfloat16)
    w_gate = (torch.randn(64, 512, device=dev) * 512 ** -0.5).to(torch.bfloat16)
    attn = torch.empty_like(q)
    proj = torch.empty(B, 512, device=dev, dtype=torch.bfloat16)
    logits = torch.empty(B, 64, device=dev, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(D)

    def step():
        FD.gqa_fwd_batch_decode(q, k, v, None, None, lens, table, scale, output_combine=attn)
        G.gemm_persistent(attn.view(B, Hq * D), w_o, out=proj)
        G.gemm_persistent(proj, w_gate, out=logits)
        return MU.topk_softmax(logits.float(), 4, True)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):          # warm-up: workspaces, function attributes, tensor-map cache
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ids_g, w_g = step()
    for trial in range(3):
        q.copy_(torch.randn(B, Hq, D, device=dev).to(torch.bfloat16))
        lens.copy_(torch.randint(1, max_len + 1, (B,), device=dev, dtype=torch.int32))
        graph.replay()
        torch.cuda.synchronize()
        check_status()
        got_attn, got_ids, got_w = attn.clone(), ids_g.clone(), w_g.clone()
        ref = FD.ref_paged_attn(q, k, v, lens, table, scale)
        torch.testing.assert_close(got_attn.float(), ref, atol=1e-2, rtol=1e-2)
        ids_e, w_e = step()           # the same ops launched eagerly on the same inputs
        torch.cuda.synchronize()
        assert torch.equal(got_ids, ids_e)
        torch.testing.assert_close(got_w, w_e, atol=0, rtol=0)
