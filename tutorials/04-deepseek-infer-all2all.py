"""Tutorial 04 — DeepSeek-style expert-parallel inference: low-latency dispatch and combine.

128 tokens per rank, hidden 7168, 256 experts, top-8 (the reference's headline configuration). One kernel
per direction:

* dispatch  quantises each token row to e4m3 with one fp32 scale per 128 values *while* copying it into the
            receive buffers of the ranks that host its experts; the per-expert counts travel in the same
            kernel and a per-source flag completes the call.
* combine   sends the experts' bf16 outputs back and reduces over top-k with the gate weights on arrival.

Buffers are double-buffered by call parity and the flags carry the call number, so calls need no barrier
between them. (reference tutorials/04-deepseek-infer-all2all.py, kernels/nvidia/low_latency_all_to_all.py)
"""
import torch

from _common import dist_print, launch
from triton_distributed_b200.ops import all_to_all as A
from triton_distributed_b200.utils import perf_func


def run(group, rank, world, dev):
    cuda = dev.type == "cuda"
    T, H, E, K = (128, 7168, 256, 8) if cuda else (16, 256, 8 * world, 2)
    ctx = A.create_moe_dispatch_context(T, H, K, E, rank, world, group=group, device=dev)
    g = torch.Generator(device="cpu").manual_seed(rank)
    x = torch.randn(T, H, generator=g).to(dev, torch.bfloat16)
    logits = torch.randn(T, E, generator=g).to(dev)
    w, ids = torch.softmax(logits, -1).topk(K, dim=-1)
    ids = ids.to(torch.int32)

    def step():
        rx, rs, splits = A.moe_dispatch(ctx, x, ids, w)
        # "experts": dequantise what arrived and hand it straight back (identity experts)
        y = A.dequant_fp8(rx, rs)
        return A.moe_combine(ctx, y, splits)

    out = step()
    # identity experts => out[t] = sum_k w[t, k] * dequant(quant(x[t]))
    q, s = A.quant_fp8_reference(x)
    ref = A.dequant_fp8(q, s).float() * w.sum(-1, keepdim=True)
    torch.testing.assert_close(out.float(), ref, atol=3e-2, rtol=3e-2)
    if cuda:
        _, ms = perf_func(step, 20, 5)
        dist_print(f"dispatch + dequant + combine: {ms * 1e3:.1f} us for {T} tokens/rank, hidden {H}, {E} experts, top-{K}")
    dist_print("dispatch/combine round trip ok")


if __name__ == "__main__":
    launch(run)
