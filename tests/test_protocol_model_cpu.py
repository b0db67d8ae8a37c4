"""The flag protocols of the fused kernels, modelled with CPU threads and C++ atomics (ranks = threads,
st.release / ld.acquire = std::memory_order_release / acquire): epoch flags with two buffer halves and no barrier
between calls, a peer that stops notifying (every waiter gives up within its limit and reports), LL packets whose
flag must EQUAL the call number (so no rank may ever run two calls ahead), the
top-bit-flip grid barrier with a changing number of participants, and the claim / copy / arrive scheme in which the
last arriver of a block publishes its flag (row staging of the grouped GEMM, sliced AG pushers). No GPU involved."""
import shutil
import subprocess
from pathlib import Path

import pytest

SRC = Path(__file__).resolve().parents[1] / "triton_distributed_b200" / "csrc" / "model" / "flag_protocol_model.cc"


@pytest.fixture(scope="module")
def model_binary(tmp_path_factory):
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        pytest.skip("no host C++ compiler")
    out = tmp_path_factory.mktemp("model") / "flag_protocol_model"
    subprocess.run([cxx, "-O2", "-std=c++17", "-pthread", str(SRC), "-o", str(out)], check=True, timeout=300)
    return out


@pytest.mark.parametrize("world,calls,seed", [(2, 300, 3), (4, 200, 1), (8, 100, 7)])
def test_flag_protocols_hold_under_random_scheduling(model_binary, world, calls, seed):
    r = subprocess.run([str(model_binary), str(world), str(calls), str(seed)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.startswith("OK")
