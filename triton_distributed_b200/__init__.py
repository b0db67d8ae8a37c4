"""Blackwell-native compute / communication overlap kernels for PyTorch.

``import triton_distributed_b200 as tdist`` gives the public names of the reference in one namespace
(``tdist.ag_gemm_intra_node``, ``tdist.fast_all_to_all``, ``tdist.SpGQAFlashDecodeAttention``, ...); the same ops are
registered with the dispatcher as ``torch.ops.tdist.*`` by :mod:`triton_distributed_b200.torch_ops`. Sub-packages:
``runtime`` (symmetric heap, process group, status block), ``ops``, ``models`` (layers and blocks), ``parallel``
(TP / SP / EP strategies), ``utils``.
"""
from . import models, ops, parallel, runtime, utils  # noqa: F401
from .models import AllGatherLayer, EPAll2AllLayer, EPMoE, SpGQAFlashDecodeAttention, TPMLP  # noqa: F401
from .ops.all_to_all import (all_to_all_post_process, create_all_to_all_context, create_moe_dispatch_context,  # noqa: F401
                             fast_all_to_all, get_ag_splits_and_recv_offset_for_dispatch,
                             get_dispatch_send_reqs_for_target_node, moe_combine, moe_dispatch, moe_expert_out_buffer)
from .ops.collectives import (AllGatherMethod, barrier_all_on_stream, cp_engine_producer_all_gather_intra_node,  # noqa: F401
                              create_fast_allgather_context, create_reduce_scater_2d_ctx, fast_allgather,
                              get_auto_all_gather_method, inter_node_allgather, reduce_scatter_2d_op,
                              reduce_scatter_ring_push_1d_intra_node_ce, reduce_scatter_ring_push_1d_intra_node_sm, ring_reduce,
                              set_signal, topk_reduce_scatter, wait_eq)
from .ops.flash_decode import (gqa_fwd_batch_decode, gqa_fwd_batch_decode_aot, gqa_fwd_batch_decode_intra_rank,  # noqa: F401
                               gqa_fwd_batch_decode_intra_rank_aot, gqa_fwd_batch_decode_persistent,
                               gqa_fwd_batch_decode_persistent_aot, inter_rank_combine,
                               kernel_inter_rank_gqa_fwd_batch_decode_combine_kv, sp_gqa_fwd_batch_decode)
from .ops.gemm import (ag_gemm_inter_node, ag_gemm_intra_node, create_ag_gemm_inter_node_context,  # noqa: F401
                       create_ag_gemm_intra_node_context, create_gemm_rs_context, gemm_non_persistent, gemm_persistent, gemm_rs,
                       gemm_rs_op)
from .ops.gemm_fp8 import (ag_gemm_fp8, create_ag_gemm_fp8_context, gemm_fp8_blockscaled, quantize_fp8_blockwise,  # noqa: F401
                           quantize_fp8_rowwise)
from .ops.moe_ep import create_ep_context, ep_combine, ep_dispatch, expert_out_buffer  # noqa: F401
from .ops.moe_tp import (ag_group_gemm_inter_node, ag_group_gemm_intra_node, create_ag_group_gemm_inter_node_context,  # noqa: F401
                         create_ag_group_gemm_intra_node_context, create_moe_rs_context, group_gemm, moe_reduce_rs,
                         select_experts, sort_topk_ids_align_block_size)
from .ops.moe_utils import bincount  # noqa: F401
from .ops.nvls import create_nvls_context, nvls_allgather, nvls_allreduce, nvls_reduce_scatter  # noqa: F401
from .runtime import TP_GROUP, check_status, finalize_distributed, initialize_distributed, symm_heap  # noqa: F401
from .runtime.dist import init_seed  # noqa: F401
from .runtime.shmem_host import (nvshmem_barrier_all, nvshmem_create_tensor, nvshmem_create_tensor_list_intra_node,  # noqa: F401
                                 nvshmem_getmem, nvshmem_int_p, nvshmem_my_pe, nvshmem_n_pes, nvshmem_p, nvshmem_ptr,
                                 nvshmem_putmem, nvshmem_team_my_pe, nvshmem_team_n_pes, nvshmemx_barrier_all_on_stream,
                                 nvshmemx_mc_ptr, nvshmemx_putmem_on_stream, nvshmemx_putmem_signal_on_stream, symm_tensor)
from .utils import (aot_compile_spaces, assert_allclose, contextual_autotune, dist_print, generate_data,  # noqa: F401
                    get_triton_combine_kv_algo_info, group_profile, perf_func)
from .utils.misc import (check_p2p_native_atomic_supported, get_has_nvlink, get_numa_world_size,  # noqa: F401
                         p2p_native_atomic_required)
