"""Host runtime: process-group bootstrap, symmetric heap, status block."""
from .dist import TP_GROUP, finalize_distributed, init_seed, initialize_distributed, set_symm_heap, symm_heap
from .heap import LocalWorld, SymmetricHeap, SymmTensor, tensor_from_ptr
from .status import StatusBlock, check_status, counters_clean, default_timeout_ns, global_status
from . import shmem_host  # noqa: E402,F401  (pynvshmem-style host API)

__all__ = [
    "TP_GROUP", "finalize_distributed", "init_seed", "initialize_distributed", "set_symm_heap", "symm_heap",
    "LocalWorld", "SymmetricHeap", "SymmTensor", "tensor_from_ptr",
    "StatusBlock", "check_status", "counters_clean", "default_timeout_ns", "global_status",
]
