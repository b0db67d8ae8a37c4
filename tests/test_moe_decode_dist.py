"""MoE all-to-all and sequence-parallel decode across ranks: gloo on CPU, native kernels on GPUs."""
import pytest
import torch

from _mp import run_workers


def test_cpu_gloo_world2():
    res, _ = run_workers("moe_decode_worker.py", 2, env={"CUDA_VISIBLE_DEVICES": ""})
    assert res["ranks_ok"] == 2 and res["fast_all_to_all"] == "ok" and res["ep_layer"] == "ok"
    assert res["fused_moe_err"] < 3e-2 and res["sp_decode_err"] < 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 8])
def test_native_on_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    res, out = run_workers("moe_decode_worker.py", world, env={"NCCL_NVLS_ENABLE": "0", "TDIST_WAIT_TIMEOUT_MS": "20000"})
    assert res["ranks_ok"] == world, out[-3000:]
