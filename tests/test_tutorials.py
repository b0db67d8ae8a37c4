"""Every tutorial runs and checks itself: as gloo ranks on CPU (the torch restatements of the ops), and on GPUs."""
import pytest
import torch

from _mp import run_workers

EXPECTED = 8


def test_tutorials_on_cpu_gloo_world2():
    res, out = run_workers("tutorials_worker.py", 2, env={"CUDA_VISIBLE_DEVICES": ""})
    assert not res["failed"], res["failed"]
    assert len(res["done"]) == EXPECTED and res["device"] == "cpu"


@pytest.mark.gpu
def test_tutorials_on_gpus():
    world = 8 if torch.cuda.device_count() >= 8 else (2 if torch.cuda.device_count() >= 2 else 1)
    res, out = run_workers("tutorials_worker.py", world, env={"NCCL_NVLS_ENABLE": "0", "TDIST_WAIT_TIMEOUT_MS": "20000"})
    assert not res["failed"], res["failed"]
    assert len(res["done"]) == EXPECTED and res["device"] == "cuda"
