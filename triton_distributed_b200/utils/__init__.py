"""Host utilities: timing, rank-filtered printing, verbose comparison, data generation, topology
probes, merged multi-rank profiling, contextual autotuning.

Counterparts of the reference's ``python/triton_dist/utils.py`` (``perf_func`` :186-198, ``dist_print``
:201-230, ``group_profile`` :282-501, ``assert_allclose`` :610-639, ``generate_data``, NVLink / NUMA
probes) and ``python/triton_dist/autotuner.py`` (``contextual_autotune``).
"""
from .aot import aot_compile_spaces, aot_spaces, get_triton_combine_kv_algo_info
from .autotuner import contextual_autotune, tunable
from .misc import (CUDA_CHECK, NvidiaSmiUtil, assert_allclose, check_p2p_native_atomic_supported, dist_print, generate_data,
                   get_has_nvlink, get_numa_node, get_numa_world_size, is_cuda, is_fp8_dtype, is_hip, p2p_bandwidth,
                   p2p_native_atomic_required, perf_func, perf_func_max_over_ranks, with_torch_deterministic)
from .config import Config
from .profile import get_torch_prof_ctx, group_profile, load_json, nvtx_range, process_trace_json

__all__ = [
    "contextual_autotune", "tunable", "assert_allclose", "check_p2p_native_atomic_supported", "dist_print",
    "generate_data", "get_has_nvlink", "get_numa_world_size", "p2p_bandwidth", "perf_func", "perf_func_max_over_ranks",
    "get_torch_prof_ctx", "group_profile", "nvtx_range", "Config", "aot_compile_spaces", "aot_spaces",
    "get_triton_combine_kv_algo_info", "p2p_native_atomic_required", "CUDA_CHECK", "NvidiaSmiUtil", "get_numa_node", "is_cuda",
    "is_fp8_dtype", "is_hip", "with_torch_deterministic", "load_json", "process_trace_json",
]
