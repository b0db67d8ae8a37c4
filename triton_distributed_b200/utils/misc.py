"""Timing, printing, comparison, data and topology helpers (see the package docstring)."""
from __future__ import annotations

import ctypes as C
import sys
from typing import Callable, Iterable, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def perf_func(func: Callable, iters: int, warmup_iters: int):
    """``(last_output, ms_per_call)`` with CUDA events around ``iters`` calls after ``warmup_iters``
    (per rank, like the reference's ``perf_func``)."""
    out = None
    for _ in range(warmup_iters):
        out = func()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        out = func()
    e1.record()
    torch.cuda.synchronize()
    return out, e0.elapsed_time(e1) / max(1, iters)


def perf_func_max_over_ranks(func: Callable, iters: int, warmup_iters: int, group=None):
    """Like :func:`perf_func` but barriers before timing and returns the slowest rank's time,
    which is what a collective op actually costs."""
    for _ in range(warmup_iters):
        func()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier(group)
        torch.cuda.synchronize()
    out, ms = perf_func(func, iters, 0)
    if dist.is_initialized():
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        ms = float(t.item())
    return out, ms


def dist_print(*args, allowed_ranks: Sequence[int] | str = (0,), prefix: bool = False, need_sync: bool = False, **kwargs):
    """``print`` on the allowed ranks only (``"all"`` = every rank); with ``need_sync`` the ranks take
    turns in rank order (one barrier per rank) so that lines do not interleave."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    allowed = range(world) if allowed_ranks == "all" else allowed_ranks
    head = (f"[rank {rank}]",) if prefix else ()
    if not need_sync or world == 1:
        if rank in allowed:
            print(*head, *args, **kwargs)
            sys.stdout.flush()
        return
    for turn in range(world):
        if turn == rank and rank in allowed:
            print(*head, *args, **kwargs)
            sys.stdout.flush()
        dist.barrier()


def assert_allclose(x: torch.Tensor, y: torch.Tensor, rtol: float = 1e-5, atol: float = 1e-8, verbose: bool = True,
                    max_print: int = 10) -> None:
    """``torch.allclose`` that, on failure, says how many elements differ, where the worst ones are
    and what both sides hold there."""
    if x.shape != y.shape:
        raise AssertionError(f"shape mismatch: {tuple(x.shape)} vs {tuple(y.shape)}")
    xf, yf = x.detach().float(), y.detach().float()
    bad = ~torch.isclose(xf, yf, rtol=rtol, atol=atol, equal_nan=True)
    nbad = int(bad.sum())
    if nbad == 0:
        return
    lines = [f"{nbad} of {x.numel()} elements differ (rtol={rtol}, atol={atol}); "
             f"max abs diff {float((xf - yf).abs().max()):.6g}"]
    if verbose:
        err = torch.where(bad, (xf - yf).abs(), torch.zeros_like(xf)).reshape(-1)
        for flat in torch.topk(err, min(max_print, nbad)).indices.tolist():
            idx = tuple(int(i) for i in torch.unravel_index(torch.tensor(flat), x.shape))
            lines.append(f"  at {idx}: {float(xf.reshape(-1)[flat]):.6g} vs {float(yf.reshape(-1)[flat]):.6g}")
    raise AssertionError("\n".join(lines))


def generate_data(configs: Iterable[Tuple[Sequence[int], torch.dtype, Tuple[float, float]]], device=None,
                  generator: Optional[torch.Generator] = None):
    """Endless generator of fresh random tensor tuples: each config is ``(shape, dtype, (scale, bias))``,
    producing ``(rand(shape) * 2 - 1) * scale + bias`` (integers: uniform in ``[-scale, scale] + bias``)."""
    device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu")
    configs = list(configs)
    while True:
        out = []
        for shape, dtype, (scale, bias) in configs:
            if dtype in (torch.int32, torch.int64, torch.int8, torch.uint8):
                t = torch.randint(int(bias - scale), int(bias + scale) + 1, tuple(shape), device=device, generator=generator).to(dtype)
            else:
                t = ((torch.rand(tuple(shape), device=device, generator=generator) * 2 - 1) * scale + bias).to(dtype)
            out.append(t)
        yield tuple(out)


# ---------------------------------------------------------------------------- topology probes
def get_has_nvlink(device: int = 0) -> bool:
    """True when the GPU has at least one active NVLink (NVML), False without NVML or a GPU."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(device)
        for link in range(18):
            try:
                if pynvml.nvmlDeviceGetNvLinkState(h, link):
                    return True
            except pynvml.NVMLError:
                break
    except Exception:  # noqa: BLE001 - no NVML, no GPU
        pass
    return False


def get_numa_world_size() -> int:
    """GPUs per NUMA domain. On an NVSwitch node every GPU reaches every peer at full bandwidth, so
    the whole node counts as one domain."""
    return torch.cuda.device_count() if torch.cuda.is_available() else 1


def check_p2p_native_atomic_supported(dev_a: int = 0, dev_b: int = 1) -> bool:
    """Whether device ``dev_a`` can run native atomics on ``dev_b``'s memory (NVLink: yes)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() <= max(dev_a, dev_b):
        return False
    try:
        rt = C.CDLL("libcudart.so.12")
    except OSError:
        return torch.cuda.can_device_access_peer(dev_a, dev_b)
    val = C.c_int(0)
    cudaDevP2PAttrNativeAtomicSupported = 3
    rc = rt.cudaDeviceGetP2PAttribute(C.byref(val), cudaDevP2PAttrNativeAtomicSupported, dev_a, dev_b)
    return rc == 0 and val.value == 1


def p2p_bandwidth(nbytes: int = 64 << 20, mode: int = 0, ctas: int = 32, threads: int = 512, chunk: int = 16384,
                  iters: int = 5, group=None) -> float:
    """GB/s of pushing (modes 0-2) / pulling (modes 3-4) ``nbytes`` to / from the next rank with the
    copy kernels of ``csrc/kernels/p2p_copy.cu``, every rank at once, slowest rank reported."""
    from .. import _lib
    from ..runtime import default_timeout_ns, global_status, symm_heap
    heap = symm_heap(group)
    rank, world = heap.rank, heap.world
    buf = heap.empty((2, nbytes), torch.uint8)
    src = torch.empty(nbytes, dtype=torch.uint8, device=buf.local.device)
    peer = (rank + 1) % world
    s, d = (src.data_ptr(), buf.peers[peer][0].data_ptr()) if mode <= 2 else (buf.peers[peer][1].data_ptr(), buf.local[0].data_ptr())
    st = global_status()

    def run():
        _lib.check(_lib.lib().tdist_p2p_copy(s, d, nbytes, mode, ctas, threads, chunk, st.device_ptr, default_timeout_ns(),
                                             torch.cuda.current_stream().cuda_stream), "tdist_p2p_copy")
    heap.barrier()
    _, ms = perf_func_max_over_ranks(run, iters, 2, group)
    heap.barrier()
    return nbytes / ms / 1e6


def p2p_native_atomic_required(fn):
    """Decorator of the reference's tests (utils.py): skip a function on systems whose peer links have no native
    atomics. NVLink always has them; the check runs only when two GPUs are visible."""
    import functools

    @functools.wraps(fn)
    def wrapped(*a, **kw):
        import torch
        if torch.cuda.is_available() and torch.cuda.device_count() >= 2 and not check_p2p_native_atomic_supported(0, 1):
            print(f"skipping {fn.__name__}: peer atomics are not native on this system")
            return None
        return fn(*a, **kw)
    return wrapped


# ---------------------------------------------------------------------------- small predicates and guards
def is_cuda() -> bool:
    """A CUDA (not ROCm) build of torch with a GPU present (reference utils.py:50-52)."""
    return bool(torch.cuda.is_available() and torch.version.hip is None)


def is_hip() -> bool:
    """Always False here: the library is sm_100a only (reference utils.py:55-57)."""
    return bool(torch.cuda.is_available() and torch.version.hip is not None)


def is_fp8_dtype(dtype: torch.dtype) -> bool:
    """One-byte floating-point types (e4m3, e5m2 and their variants); reference utils.py:130-131."""
    return dtype.is_floating_point and torch.empty((), dtype=dtype).element_size() == 1


class with_torch_deterministic:
    """``with with_torch_deterministic(True): ...`` switches torch's deterministic-algorithms mode for the block and
    puts the previous mode back afterwards, also when the block raises (reference utils.py:121-127). Also usable as a
    decorator."""

    def __init__(self, mode: bool, warn_only: bool = True):
        self.mode, self.warn_only = mode, warn_only

    def __enter__(self):
        self._old = torch.are_deterministic_algorithms_enabled()
        self._old_warn = torch.is_deterministic_algorithms_warn_only_enabled()
        torch.use_deterministic_algorithms(self.mode, warn_only=self.warn_only)
        return self

    def __exit__(self, *exc):
        torch.use_deterministic_algorithms(self._old, warn_only=self._old_warn)
        return False

    def __call__(self, fn):
        import functools

        @functools.wraps(fn)
        def wrapper(*a, **kw):
            with with_torch_deterministic(self.mode, self.warn_only):
                return fn(*a, **kw)
        return wrapper


def CUDA_CHECK(err):
    """Raise unless ``err`` is a success code. Accepts what cuda-python calls return (a result enum, or a tuple whose
    first element is one: the rest of the tuple is handed back), a plain integer, or a ``tdist`` return code
    (reference utils.py:233-241)."""
    rest = None
    if isinstance(err, tuple):
        err, rest = err[0], err[1:]
    code = int(getattr(err, "value", err))
    if code != 0:
        name = getattr(err, "name", None) or str(err)
        raise RuntimeError(f"CUDA error {code}: {name}")
    if rest is None:
        return None
    return rest[0] if len(rest) == 1 else rest


# ---------------------------------------------------------------------------- topology from nvidia-smi / sysfs
class NvidiaSmiUtil:
    """Topology facts read from ``nvidia-smi`` text and sysfs, for hosts without NVML bindings (reference
    utils.py:504-544). The parsers take the text as an argument so that they can be checked without a GPU."""

    @staticmethod
    def parse_topo_matrix(text: str):
        """``nvidia-smi topo -m`` output -> square matrix with 1 where two GPUs are linked by NVLink (``NV<n>``), 0 on
        the diagonal, -1 otherwise."""
        rows = [ln.split() for ln in text.splitlines() if ln.startswith("GPU") and len(ln.split()) > 1 and ln.split()[0][3:].isdigit()]
        n = len(rows)
        out = [[-1] * n for _ in range(n)]
        for i, cols in enumerate(rows):
            for j in range(n):
                cell = cols[1 + j] if 1 + j < len(cols) else ""
                out[i][j] = 0 if cell == "X" else (1 if cell.startswith("NV") else -1)
        return out

    @staticmethod
    def get_nvlink_adjacency_matrix():
        import subprocess
        return NvidiaSmiUtil.parse_topo_matrix(subprocess.check_output(["nvidia-smi", "topo", "-m"], text=True, timeout=30))

    @staticmethod
    def numa_node_of_bus_id(bus_id: str, sysfs_root: str = "/sys/bus/pci/devices") -> int:
        """NUMA node of the PCI device ``bus_id`` (``00000000:17:00.0`` as nvidia-smi prints it); -1 when unknown."""
        import os
        short = bus_id.strip().lower()
        if short.count(":") == 2 and len(short.split(":")[0]) == 8:
            short = short[4:]                       # 8-digit domain -> the 4 digits sysfs uses
        try:
            with open(os.path.join(sysfs_root, short, "numa_node")) as f:
                return max(int(f.read().strip()), 0)
        except (OSError, ValueError):
            return -1

    @staticmethod
    def get_gpu_numa_node(gpu_index: int = 0) -> int:
        import subprocess
        try:
            bus = subprocess.check_output(["nvidia-smi", "--query-gpu=pci.bus_id", "--format=csv,noheader,nounits", "-i", str(gpu_index)],
                                          text=True, timeout=30)
        except (OSError, subprocess.SubprocessError):
            return -1
        return NvidiaSmiUtil.numa_node_of_bus_id(bus)


def get_numa_node(gpu_index: int = 0) -> int:
    """NUMA node the GPU hangs off: NVML when it knows, else nvidia-smi + sysfs, else -1 (reference utils.py:581-586)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        return int(pynvml.nvmlDeviceGetNumaNodeId(pynvml.nvmlDeviceGetHandleByIndex(gpu_index)))
    except Exception:  # noqa: BLE001 - no NVML, old driver, no GPU
        return NvidiaSmiUtil.get_gpu_numa_node(gpu_index)
