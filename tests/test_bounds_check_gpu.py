"""The bounds-checked build of the library: peer-index and span checks in the symmetric-address helpers."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_out_of_range_accesses_are_recorded_and_skipped(cuda_device):
    env = dict(os.environ, TDIST_BOUNDS_CHECK="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "workers", "bounds_worker.py")], capture_output=True, text=True,
                          timeout=300, env=env, cwd=ROOT)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    res = json.loads([line for line in proc.stdout.splitlines() if line.startswith("RESULT ")][-1][len("RESULT "):])
    assert res["checked_lib"] and res["path"] == "libtdist_check.so"
    assert res["in_range_ok"]
    assert res["skipped"] == 3
    assert "bad argument" in res["raised"] and "bounds check" in res["raised"]
    assert res["memory_untouched"] and res["usable_after"]


@pytest.mark.gpu
def test_the_regular_build_refuses_the_probe(cuda_device):
    from triton_distributed_b200 import _lib
    from triton_distributed_b200.ops import primitives as P
    from triton_distributed_b200.runtime import LocalWorld

    if _lib.bounds_checked():
        pytest.skip("this process runs the checked build")
    lw = LocalWorld(1, cuda_device)
    ctx = P.create_primitive_context(0, 1, 256, heap=lw.heap(0))
    with pytest.raises(_lib.TdistError, match="bounds-checked build"):
        P.run_primitive(ctx, "bounds_probe")
