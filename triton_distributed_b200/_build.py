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


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".h", ".cuh", ".hpp"):
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, hdr_digest: str, verbose: bool) -> tuple[Path, bool, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".sha")
    digest = hashlib.sha256(src.read_bytes() + hdr_digest.encode()).hexdigest()
    if obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj, False, ""
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = proc.stdout + proc.stderr
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{log}")
    (OBJ_DIR / (src.stem + ".ptxas.txt")).write_text(log)
    stamp.write_text(digest)
    if verbose:
        print(f"[tdist build] compiled {src.name}", file=sys.stderr)
    return obj, True, log


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every source for sm_100a and link ``libtdist.so``. Returns its path."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for p in OBJ_DIR.glob("*.sha"):
            p.unlink()
    hdr = _headers_digest()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as ex:
        results = list(ex.map(lambda s: _compile_one(nvcc, s, hdr, verbose), srcs))
    objs = [r[0] for r in results]
    changed = any(r[1] for r in results)
    # drop objects whose source disappeared
    keep = {o.name for o in objs}
    for o in OBJ_DIR.glob("*.o"):
        if o.name not in keep:
            o.unlink()
            changed = True
    if changed or not LIB_PATH.exists():
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-ldl", "-lpthread"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}{proc.stderr}")
        if verbose:
            print(f"[tdist build] linked {LIB_PATH}", file=sys.stderr)
    return LIB_PATH


def ptxas_report() -> str:
    """Concatenated ``-Xptxas -v`` output of the last compilation of every source."""
    return "\n".join(p.read_text() for p in sorted(OBJ_DIR.glob("*.ptxas.txt")))


if __name__ == "__main__":
    path = build(verbose=True, force="--force" in sys.argv)
    print(path)
