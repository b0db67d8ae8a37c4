"""Tensor-parallel MoE ops across ranks: gloo on CPU (world 2) and NCCL on GPUs, every launch mode."""
import pytest
import torch

from _mp import run_workers


def test_cpu_gloo_world2():
    res, _ = run_workers("moe_tp_worker.py", 2, env={"CUDA_VISIBLE_DEVICES": ""})
    assert res["world"] == 2 and res["ranks_ok"] == 2 and res["device"] == "cpu"
    assert res["ag_group_gemm_max_err"] < 1e-3 and res["moe_reduce_rs_max_err"] < 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_moe_tp_ops_on_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    res, out = run_workers("moe_tp_worker.py", world, env={"NCCL_NVLS_ENABLE": "0", "TDIST_WAIT_TIMEOUT_MS": "20000"})
    assert res["ranks_ok"] == world, out[-3000:]
    assert res["modes"] == ["fused", "staged", "cp_async"]
    assert res["ag_group_gemm_max_err"] < 0.1 and res["moe_reduce_rs_max_err"] < 0.2
