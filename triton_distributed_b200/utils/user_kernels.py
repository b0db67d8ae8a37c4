"""Build and load kernels that users write against the device headers of this library.

The reference's primitives are a Python-embedded device language: a user writes a Triton kernel that calls
``dl.wait`` / ``dl.notify`` / ``libshmem_device.putmem_signal_block`` and the patched compiler lowers them
(reference python/triton_dist/language.py:57-112, tutorials/01-distributed-notify-wait.py:64-133). Here the
primitives are CUDA device functions in header files (``csrc/device/signal.cuh``, ``shmem.cuh``, ``ll.cuh``,
``ptx.cuh``, ``language_extra.cuh``); a user kernel is a ``.cu`` file that includes them, compiled for sm_100a with
nvcc into a shared library next to its source and called through ``ctypes``:

    lib = load_user_library("my_kernels.cu")            # builds <dir>/_build/libmy_kernels.so when the source changed
    lib.my_launch(symm.ptr_array(), rank, world, ...)

The ``extern "C"`` launchers of such a file take raw pointers: a symmetric tensor is passed as the array of its
per-rank addresses (``SymmTensor.ptr_array()``), from which the launcher fills a ``tdist::SymmWindow``.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import subprocess
from pathlib import Path
from typing import Iterable, Sequence, Union

from .. import _build

INCLUDE_DIR = _build.CSRC          # user sources write  #include "device/signal.cuh"


def _digest(sources: Sequence[Path], flags: Sequence[str]) -> str:
    h = hashlib.sha256(_build._headers_digest(flags).encode())
    for s in sources:
        h.update(s.read_bytes())
    return h.hexdigest()


def build_user_library(sources: Union[str, Path, Iterable[Union[str, Path]]], name: str = "", extra_flags: Sequence[str] = (),
                       verbose: bool = False) -> Path:
    """Compile ``sources`` (``.cu`` files) for sm_100a into ``<dir of the first source>/_build/lib<name>.so`` unless an
    up-to-date build is there already. Returns the library's path."""
    if isinstance(sources, (str, Path)):
        sources = [sources]
    srcs = [Path(s).resolve() for s in sources]
    name = name or srcs[0].stem
    out_dir = srcs[0].parent / "_build"
    lib = out_dir / f"lib{name}.so"
    stamp = out_dir / f"lib{name}.sha"
    flags = list(extra_flags)
    digest = _digest(srcs, flags)
    if lib.exists() and stamp.exists() and stamp.read_text() == digest:
        return lib
    out_dir.mkdir(parents=True, exist_ok=True)
    cmd = [_build._nvcc(), *_build.ARCH_FLAGS, *_build.NVCC_FLAGS, *flags, f"-I{INCLUDE_DIR}", "-shared", "-o", str(lib),
           *map(str, srcs)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {name}:\n{proc.stdout}{proc.stderr}")
    stamp.write_text(digest)
    if verbose:
        print(f"[tdist build] built {lib}")
    return lib


def load_user_library(sources, name: str = "", extra_flags: Sequence[str] = ()) -> C.CDLL:
    """:func:`build_user_library`, then ``ctypes.CDLL`` of the result."""
    return C.CDLL(str(build_user_library(sources, name, extra_flags)))
