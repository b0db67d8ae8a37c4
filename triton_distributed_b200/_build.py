"""In-tree build of ``libtdist.so`` for sm_100a.

The native code has no PyTorch dependency (raw device pointers and streams cross the C ABI),
so it is compiled with plain ``nvcc``: every ``.cu`` / ``.cc`` under ``csrc/`` becomes an object
under ``_C/obj`` and the objects are linked into ``_C/libtdist.so``. Objects are rebuilt only
when their source, one of the headers, or the flags changed (content hash).

Plays the role of the reference's CMake + ``setup.py`` tree (reference python/setup.py:589-768,
csrc/CMakeLists.txt), which builds ``libtriton_distributed.so`` and ``_pynvshmem``.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OUT_DIR = PKG_DIR / "_C"
OBJ_DIR = OUT_DIR / "obj"
LIB_PATH = OUT_DIR / "libtdist.so"
# the same sources with -DTDIST_BOUNDS_CHECK: every symmetric-address translation checks peer and span, records the
# first violation and skips the access (csrc/device/signal.cuh); loaded instead of the above with TDIST_BOUNDS_CHECK=1
CHECK_OBJ_DIR = OUT_DIR / "obj_check"
CHECK_LIB_PATH = OUT_DIR / "libtdist_check.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-Wall", "-Xcompiler", "-Wno-unknown-pragmas", "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("TDIST_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set TDIST_NVCC)")


def sources() -> list[Path]:
    out = []
    for sub in ("runtime", "kernels"):
        out += sorted((CSRC / sub).glob("*.cu")) + sorted((CSRC / sub).glob("*.cc"))
    return out


def _headers_digest(extra_flags=()) -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".h", ".cuh", ".hpp"):
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join([*ARCH_FLAGS, *NVCC_FLAGS, *extra_flags]).encode())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, hdr_digest: str, verbose: bool, obj_dir: Path = OBJ_DIR, extra_flags=()) -> tuple[Path, bool, str]:
    obj = obj_dir / (src.stem + ".o")
    stamp = obj_dir / (src.stem + ".sha")
    digest = hashlib.sha256(src.read_bytes() + hdr_digest.encode()).hexdigest()
    if obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj, False, ""
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *extra_flags, "-x", "cu", "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = proc.stdout + proc.stderr
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{log}")
    (obj_dir / (src.stem + ".ptxas.txt")).write_text(log)
    stamp.write_text(digest)
    if verbose:
        print(f"[tdist build] compiled {src.name}" + (f" ({' '.join(extra_flags)})" if extra_flags else ""), file=sys.stderr)
    return obj, True, log


def _build_variant(lib_path: Path, obj_dir: Path, extra_flags, verbose: bool, force: bool) -> Path:
    nvcc = _nvcc()
    obj_dir.mkdir(parents=True, exist_ok=True)
    if force:
        for p in obj_dir.glob("*.sha"):
            p.unlink()
    hdr = _headers_digest(extra_flags)
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as ex:
        results = list(ex.map(lambda s: _compile_one(nvcc, s, hdr, verbose, obj_dir, extra_flags), srcs))
    objs = [r[0] for r in results]
    changed = any(r[1] for r in results)
    # drop objects whose source disappeared
    keep = {o.name for o in objs}
    for o in obj_dir.glob("*.o"):
        if o.name not in keep:
            o.unlink()
            changed = True
    if changed or not lib_path.exists():
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(lib_path), *map(str, objs), "-ldl", "-lpthread"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}{proc.stderr}")
        if verbose:
            print(f"[tdist build] linked {lib_path}", file=sys.stderr)
    return lib_path


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every source for sm_100a and link ``libtdist.so`` (and its bounds-checked twin
    ``libtdist_check.so``). Returns the path of the former."""
    path = _build_variant(LIB_PATH, OBJ_DIR, (), verbose, force)
    _build_variant(CHECK_LIB_PATH, CHECK_OBJ_DIR, ("-DTDIST_BOUNDS_CHECK",), verbose, force)
    return path


def ptxas_report() -> str:
    """Concatenated ``-Xptxas -v`` output of the last compilation of every source."""
    return "\n".join(p.read_text() for p in sorted(OBJ_DIR.glob("*.ptxas.txt")))


if __name__ == "__main__":
    path = build(verbose=True, force="--force" in sys.argv)
    print(path)
