"""NVLS (multimem) all-gather / reduce-scatter / all-reduce: gloo world 2 for the plumbing, GPUs for the kernels."""
import pytest
import torch

from _mp import run_workers


def test_cpu_gloo_world2_plumbing():
    res, out = run_workers("nvls_worker.py", 2, env={"CUDA_VISIBLE_DEVICES": ""})
    assert res["ranks_ok"] == 2 and res["checked"], out[-2000:]


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 8])
def test_multimem_collectives_on_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    res, out = run_workers("nvls_worker.py", world, env={"TDIST_NVLS": "1", "TDIST_WAIT_TIMEOUT_MS": "20000"})
    assert res["ranks_ok"] == world, out[-3000:]
    if not res["multicast"]:
        pytest.skip("this system offers no NVLS multicast objects")
    assert res["checked"] and res["fast_allgather_used_nvls"] and res["sp_decode_multicast"]
