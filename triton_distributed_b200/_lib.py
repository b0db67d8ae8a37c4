"""ctypes binding of ``libtdist.so`` (the C ABI is declared in ``csrc/include/tdist.h``).

The library is built in-tree by :mod:`triton_distributed_b200._build`. On a machine with a GPU
a missing or unloadable library is an error, never a silent fallback: ops that need native code
call :func:`lib` and raise.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

MAX_RANKS = 8

_LIB = None
_LOCK = threading.Lock()


class TdistError(RuntimeError):
    """A native entry point returned a non-zero code."""


class TdistTimeoutError(TdistError):
    """A bounded device-side wait gave up; the status block says which."""


class Status(C.Structure):
    _fields_ = [
        ("abort_flag", C.c_int), ("code", C.c_int), ("kernel_id", C.c_int), ("rank", C.c_int),
        ("peer", C.c_int), ("index", C.c_int), ("expected", C.c_longlong), ("seen", C.c_longlong),
        ("block", C.c_int), ("where", C.c_int), ("reserved", C.c_int * 4),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p),
        ("a_ws", C.c_void_p),
        ("a_ws_peer", C.c_void_p * MAX_RANKS),
        ("b", C.c_void_p),
        ("c", C.c_void_p),
        ("c_stage_peer", C.c_void_p * MAX_RANKS),
        ("rs_out", C.c_void_p),
        ("flags", C.c_void_p),
        ("flags_peer", C.c_void_p * MAX_RANKS),
        ("m_per_rank", C.c_int), ("n", C.c_int), ("k", C.c_int),
        ("world", C.c_int), ("rank", C.c_int),
        ("mode", C.c_int), ("dtype", C.c_int),
        ("epoch", C.c_uint32),
        ("num_sms", C.c_int), ("num_comm_sms", C.c_int), ("debug_delay_ns", C.c_int), ("group_m", C.c_int), ("cta_pair", C.c_int),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("stream", C.c_void_p),
        ("trace", C.c_void_p),
        ("expert_ids", C.c_void_p), ("num_m_blocks", C.c_void_p), ("num_experts", C.c_int),
        ("a_ws_mc", C.c_void_p), ("push_count", C.c_void_p),
        ("a_gather", C.c_void_p), ("a_gather_rows", C.c_int), ("block_src", C.c_void_p), ("src_flags", C.c_void_p),
        ("src_epoch", C.c_uint64), ("src_rank", C.c_int), ("src_world", C.c_int),
        ("gather_dst", C.c_void_p), ("block_ready", C.c_void_p), ("gather_counter", C.c_void_p), ("block_rot", C.c_void_p),
        ("c_scatter", C.c_void_p), ("c_rows", C.c_int),
    ]


class GemmFp8Args(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("sa", C.c_void_p), ("b", C.c_void_p), ("sb", C.c_void_p), ("c", C.c_void_p),
        ("a_ws", C.c_void_p), ("sa_ws", C.c_void_p),
        ("a_ws_peer", C.c_void_p * MAX_RANKS), ("sa_ws_peer", C.c_void_p * MAX_RANKS),
        ("flags", C.c_void_p), ("flags_peer", C.c_void_p * MAX_RANKS),
        ("m_per_rank", C.c_int), ("n", C.c_int), ("k", C.c_int),
        ("world", C.c_int), ("rank", C.c_int), ("mode", C.c_int),
        ("epoch", C.c_uint32),
        ("num_sms", C.c_int), ("num_comm_sms", C.c_int),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("stream", C.c_void_p),
    ]


class NvlsArgs(C.Structure):
    _fields_ = [
        ("mc", C.c_void_p), ("local", C.c_void_p),
        ("sig_peer", C.c_void_p * MAX_RANKS),
        ("counters", C.c_void_p), ("output", C.c_void_p),
        ("seg_bytes", C.c_size_t),
        ("world", C.c_int), ("rank", C.c_int), ("op", C.c_int), ("dtype", C.c_int), ("ctas", C.c_int),
        ("epoch", C.c_uint64),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("stream", C.c_void_p),
    ]


class CollArgs(C.Structure):
    _fields_ = [
        ("buf_peer", C.c_void_p * MAX_RANKS),
        ("sig_peer", C.c_void_p * MAX_RANKS),
        ("ll_peer", C.c_void_p * MAX_RANKS),
        ("counters", C.c_void_p),
        ("input", C.c_void_p),
        ("output", C.c_void_p),
        ("seg_bytes", C.c_size_t),
        ("world", C.c_int), ("rank", C.c_int),
        ("mode", C.c_int), ("phase", C.c_int), ("ctas_per_peer", C.c_int), ("dtype", C.c_int),
        ("epoch", C.c_uint64),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("stream", C.c_void_p),
        ("pos_of", C.c_void_p), ("topk_w", C.c_void_p), ("topk", C.c_int), ("row_bytes", C.c_int),
    ]


class A2AArgs(C.Structure):
    _fields_ = [
        ("send", C.c_void_p), ("src_index", C.c_void_p), ("counts", C.c_void_p), ("send_scale", C.c_void_p),
        ("recv_peer", C.c_void_p * MAX_RANKS), ("scale_peer", C.c_void_p * MAX_RANKS),
        ("splits_peer", C.c_void_p * MAX_RANKS), ("sig_peer", C.c_void_p * MAX_RANKS),
        ("counters", C.c_void_p),
        ("slot_of", C.c_void_p), ("cumsum", C.c_void_p), ("topk_ids", C.c_void_p), ("topk_w", C.c_void_p),
        ("out", C.c_void_p),
        ("ntok", C.c_int), ("topk", C.c_int),
        ("row_bytes_in", C.c_int), ("row_bytes_out", C.c_int), ("scale_cols", C.c_int), ("hidden", C.c_int),
        ("max_m", C.c_int), ("epr", C.c_int), ("world", C.c_int), ("rank", C.c_int),
        ("mode", C.c_int), ("quant", C.c_int), ("reduce", C.c_int), ("phase", C.c_int), ("ctas_per_peer", C.c_int),
        ("epoch", C.c_uint64),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("stream", C.c_void_p),
    ]


class MoeDispatchArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("topk_ids", C.c_void_p), ("slot_of", C.c_void_p), ("cumsum", C.c_void_p),
        ("recv_peer", C.c_void_p * MAX_RANKS), ("scale_peer", C.c_void_p * MAX_RANKS),
        ("counts_peer", C.c_void_p * MAX_RANKS), ("sig_peer", C.c_void_p * MAX_RANKS),
        ("counters", C.c_void_p), ("pair_row", C.c_void_p), ("send_splits", C.c_void_p), ("recv_splits", C.c_void_p),
        ("recv_offset", C.c_void_p), ("num_recv", C.c_void_p), ("block_expert", C.c_void_p), ("num_blocks", C.c_void_p),
        ("ntok", C.c_int), ("topk", C.c_int), ("hidden", C.c_int), ("num_experts", C.c_int), ("world", C.c_int), ("rank", C.c_int),
        ("max_m", C.c_int), ("quant", C.c_int), ("compact", C.c_int), ("align", C.c_int), ("phase", C.c_int), ("num_ctas", C.c_int),
        ("epoch", C.c_uint64),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("stream", C.c_void_p),
    ]


class MoeCombineArgs(C.Structure):
    _fields_ = [
        ("buf_peer", C.c_void_p * MAX_RANKS), ("sig_peer", C.c_void_p * MAX_RANKS),
        ("topk_ids", C.c_void_p), ("topk_w", C.c_void_p), ("pair_row", C.c_void_p), ("out", C.c_void_p),
        ("ntok", C.c_int), ("topk", C.c_int), ("hidden", C.c_int), ("epr", C.c_int), ("world", C.c_int), ("rank", C.c_int),
        ("phase", C.c_int), ("num_ctas", C.c_int),
        ("epoch", C.c_uint64),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("stream", C.c_void_p),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("block_table", C.c_void_p),
        ("kv_lens", C.c_void_p), ("partial", C.c_void_p), ("counters", C.c_void_p), ("out", C.c_void_p),
        ("ll_peer", C.c_void_p * MAX_RANKS),
        ("B", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int), ("head_dim", C.c_int), ("page_size", C.c_int),
        ("max_blocks", C.c_int), ("splits", C.c_int),
        ("stride_block", C.c_longlong), ("stride_token", C.c_longlong), ("stride_head", C.c_longlong),
        ("scale", C.c_float), ("soft_cap", C.c_float),
        ("mode", C.c_int), ("dtype", C.c_int), ("world", C.c_int), ("rank", C.c_int),
        ("epoch", C.c_uint32), ("push_only", C.c_int),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("stream", C.c_void_p),
        ("epoch_ptr", C.c_void_p), ("epoch_done", C.c_void_p), ("ll_peer_alt", C.c_void_p * MAX_RANKS),
        ("ll_mc", C.c_void_p), ("ll_mc_alt", C.c_void_p),
    ]


class PrimArgs(C.Structure):
    _fields_ = [
        ("data_peer", C.c_void_p * MAX_RANKS), ("sig_peer", C.c_void_p * MAX_RANKS),
        ("result", C.c_void_p), ("grid_counter", C.c_void_p), ("barrier_epoch", C.c_void_p),
        ("world", C.c_int), ("rank", C.c_int), ("op", C.c_int), ("phase", C.c_int), ("nbytes", C.c_int),
        ("scope", C.c_int), ("grid", C.c_int),
        ("value", C.c_uint64),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("stream", C.c_void_p),
    ]


(PRIM_RING_PUT, PRIM_NOTIFY_WAIT, PRIM_NOTIFY_ADD, PRIM_PUT_SIGNAL, PRIM_PUT_QUIET_SIGNAL, PRIM_GET, PRIM_BROADCAST,
 PRIM_FCOLLECT, PRIM_GRID_BARRIER, PRIM_SCOPED_OPS, PRIM_BARRIER, PRIM_BOUNDS_PROBE) = range(12)
GEMM_PLAIN, GEMM_AG, GEMM_RS = 0, 1, 2
A2A_DISPATCH, A2A_COMBINE = 0, 1
DT_BF16, DT_F16, DT_F32, DT_I32 = 0, 1, 2, 3
AG_PULL, AG_PUSH, AG_LL, AG_PUSH_ORDERED = 0, 1, 2, 3


def bounds_checked() -> bool:
    """True when ``TDIST_BOUNDS_CHECK=1`` selects the library whose symmetric-address translation checks peer and
    span, records the first violation in the status block and skips the access (read once, at load time)."""
    return os.environ.get("TDIST_BOUNDS_CHECK", "0") == "1"


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "_C" / ("libtdist_check.so" if bounds_checked() else "libtdist.so")


def available() -> bool:
    return lib_path().exists()


def _declare(lib):
    lib.tdist_last_error.restype = C.c_char_p
    lib.tdist_last_error.argtypes = []
    lib.tdist_status_create.argtypes = [C.POINTER(C.c_void_p)]
    lib.tdist_status_read.argtypes = [C.c_void_p, C.POINTER(Status)]
    lib.tdist_status_reset.argtypes = [C.c_void_p]
    lib.tdist_status_destroy.argtypes = [C.c_void_p]
    lib.tdist_gemm_run.argtypes = [C.POINTER(GemmArgs)]
    lib.tdist_gemm_grid.argtypes = [C.POINTER(GemmArgs)]
    lib.tdist_gemm_plan.argtypes = [C.POINTER(GemmArgs), C.POINTER(C.c_int)]
    lib.tdist_gemm_plan.restype = C.c_int
    lib.tdist_gemm_schedule_check.argtypes = [C.c_int] * 8 + [C.POINTER(C.c_int), C.POINTER(C.c_int)]
    lib.tdist_gemm_schedule_check.restype = C.c_int
    lib.tdist_gemm_fp8_run.argtypes = [C.POINTER(GemmFp8Args)]
    lib.tdist_allgather.argtypes = [C.POINTER(CollArgs)]
    lib.tdist_nvls.argtypes = [C.POINTER(NvlsArgs)]
    lib.tdist_reduce_scatter.argtypes = [C.POINTER(CollArgs)]
    lib.tdist_ring_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.tdist_barrier_all.argtypes = [C.POINTER(C.c_void_p), C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_uint64, C.c_void_p]
    lib.tdist_p2p_copy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.c_void_p, C.c_uint64, C.c_void_p]
    lib.tdist_a2a.argtypes = [C.POINTER(A2AArgs)]
    lib.tdist_moe_dispatch.argtypes = [C.POINTER(MoeDispatchArgs)]
    lib.tdist_moe_combine.argtypes = [C.POINTER(MoeCombineArgs)]
    lib.tdist_signal_op_on_stream.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_void_p]
    lib.tdist_signal_wait_on_stream.argtypes = [C.c_void_p, C.c_int, C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p]
    lib.tdist_primitive.argtypes = [C.POINTER(PrimArgs)]
    lib.tdist_bounds_checked.argtypes = []
    lib.tdist_flash_decode.argtypes = [C.POINTER(DecodeArgs)]
    lib.tdist_lse_combine.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    lib.tdist_dequant_fp8.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    lib.tdist_moe_route.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_void_p]
    lib.tdist_moe_align_block_size.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                               C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.tdist_gather_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.tdist_topk_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    lib.tdist_moe_topk_softmax.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.tdist_stream_write_value.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_int]
    lib.tdist_stream_wait_value.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_int, C.c_int]


def lib():
    """Load (once) and return the native library; build it first if sources are newer."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = lib_path()
        if not path.exists() or os.environ.get("TDIST_REBUILD") == "1":
            from . import _build
            _build.build()
        if not path.exists():
            raise TdistError(f"native library missing: {path} (run python -m triton_distributed_b200._build)")
        handle = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
        _declare(handle)
        _LIB = handle
    return _LIB


def check(code: int, what: str = "") -> None:
    if code == 0:
        return
    msg = lib().tdist_last_error().decode(errors="replace")
    raise TdistError(f"{what or 'native call'} failed with code {code}: {msg}")


def ptr_array(values) -> "C.Array":
    arr = (C.c_void_p * MAX_RANKS)()
    for i, v in enumerate(values):
        arr[i] = int(v) if v else None
    return arr
