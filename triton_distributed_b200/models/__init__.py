"""Layer-level wrappers (the reference's ``python/triton_dist/layers/nvidia``) and the small model
blocks the benchmarks and smoke tests drive: a tensor-parallel MLP (AG-GEMM -> activation -> GEMM-RS)
and an expert-parallel MoE block (fp8 dispatch -> grouped expert GEMMs -> weighted combine)."""
from .layers import AllGatherLayer, EPAll2AllLayer, SpGQAFlashDecodeAttention
from .blocks import EPMoE, TPMLP

__all__ = ["AllGatherLayer", "EPAll2AllLayer", "SpGQAFlashDecodeAttention", "EPMoE", "TPMLP"]
