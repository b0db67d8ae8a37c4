"""Barrier / all-gather / reduce-scatter across ranks: gloo on CPU, the native kernels on GPUs."""
import pytest
import torch

from _mp import run_workers


def test_cpu_gloo_world2():
    res, _ = run_workers("collectives_worker.py", 2, env={"CUDA_VISIBLE_DEVICES": ""})
    assert res["ranks_ok"] == 2 and res["reduce_scatter"] == "ok"


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 8])
def test_native_collectives_on_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    res, out = run_workers("collectives_worker.py", world, env={"NCCL_NVLS_ENABLE": "0", "TDIST_WAIT_TIMEOUT_MS": "20000"})
    assert res["ranks_ok"] == world, out[-3000:]
    assert res["barrier"] == "ok"
