"""Op library (tensor-parallel GEMMs, collectives, MoE all-to-all, flash decode)."""
from .gemm import (AllGatherGEMMTensorParallelContext, GEMMReduceScatterTensorParallelContext, ag_gemm_intra_node,
                   create_ag_gemm_intra_node_context, create_gemm_rs_context, gemm_non_persistent, gemm_persistent,
                   gemm_rs)
from .gemm_fp8 import (AGGemmFp8Context, ag_gemm_fp8, create_ag_gemm_fp8_context, dequantize_fp8, gemm_fp8_blockscaled,
                       quantize_fp8_blockwise, quantize_fp8_rowwise)
