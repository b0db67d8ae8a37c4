"""Op library (tensor-parallel GEMMs, collectives, MoE all-to-all, flash decode)."""
from .gemm import (AllGatherGEMMTensorParallelContext, GEMMReduceScatterTensorParallelContext, ag_gemm_intra_node,
                   create_ag_gemm_intra_node_context, create_gemm_rs_context, gemm_non_persistent, gemm_persistent,
                   gemm_rs)
