"""AG-GEMM / GEMM-RS across ranks: gloo on CPU (world 2, fp32, rtol 1e-5) and NCCL on GPUs."""
import pytest
import torch

from _mp import run_workers


def test_cpu_gloo_world2_plumbing():
    res, _ = run_workers("tp_gemm_worker.py", 2, env={"CUDA_VISIBLE_DEVICES": ""})
    assert res["world"] == 2 and res["ranks_ok"] == 2 and res["device"] == "cpu"
    assert res["ag_max_err"] < 1e-4 and res["rs_max_err"] < 1e-4
    assert res["fp8_ag_max_err"] < 0.05


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_ops_on_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    res, out = run_workers("tp_gemm_worker.py", world, env={"NCCL_NVLS_ENABLE": "0", "TDIST_WAIT_TIMEOUT_MS": "20000"})
    assert res["ranks_ok"] == world, out[-3000:]
    assert res["ag_max_err"] < 0.1 and res["rs_max_err"] < 0.1 and res["fp8_ag_max_err"] < 0.2


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 8])
def test_ag_gemm_with_multicast_pushers(world):
    """The same worker with the heap bound to an NVSwitch multicast object: the AG-GEMM pushers store each
    block once with multimem.st instead of once per peer."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    res, out = run_workers("tp_gemm_worker.py", world, env={"NCCL_NVLS_ENABLE": "0", "TDIST_NVLS": "1", "TDIST_AG_GEMM_NVLS": "2", "TDIST_WAIT_TIMEOUT_MS": "20000"})
    assert res["ranks_ok"] == world, out[-3000:]
    if not res["ag_multicast_pusher"]:
        pytest.skip("this system offers no NVLS multicast objects")
    assert res["ag_max_err"] < 0.1 and res["rs_max_err"] < 0.1
