"""The autotuner over the ops' real knobs, across ranks (gloo, CPU)."""
from _mp import run_workers

from triton_distributed_b200.ops import tuned as TU


def test_all_ranks_pick_the_same_ag_gemm_config(tmp_path):
    res, out = run_workers("autotune_worker.py", 2, env={"CUDA_VISIBLE_DEVICES": "", "TDIST_TEST_TMP": str(tmp_path)}, timeout=300)
    assert res is not None, out[-2000:]
    space = TU.AG_GEMM_SPACE
    for r in res:
        assert r["ok"] and r["restored"], res
        assert r["picked"] == [space[5]], res                      # the best of the per-config maxima, on both ranks
        assert r["measured"] >= len(space) * 3 and r["after"] == 1, res   # once tuned, a step is one plain call
    assert (tmp_path / ".autotune_logs" / "rank-1.log").exists()


def test_tuned_spaces_start_with_the_launchers_own_choice():
    # outside a tuning session the wrappers run configuration 0: that must be "let the launcher decide"
    assert TU.AG_GEMM_SPACE[0] == {"num_comm_sms": 0, "cta_pair": -1}
    assert TU.GEMM_RS_SPACE[0] == {"cta_pair": -1}
    assert TU.DECODE_SPACE[0] == {"kv_split": -1}
    assert TU.MOE_DISPATCH_SPACE[0] == {"num_ctas": 0}
