"""Failure detection without a GPU fault: failures are made on the host (a rank that leaves, a bad descriptor)
and every waiter must notice within a limit and say so."""
import os
import socket

import pytest

from _mp import run_workers


def test_a_rank_that_leaves_is_detected_by_the_others():
    res, out = run_workers("failure_worker.py", 2, env={"CUDA_VISIBLE_DEVICES": "", "TDIST_TEST_PG_TIMEOUT_S": "5"}, timeout=120)
    assert res is not None and res["detected"], out[-2000:]
    assert res["seconds"] < 60, res


def test_descriptor_exchange_refuses_a_bad_descriptor():
    """The heap's descriptor exchange (SCM_RIGHTS over a Unix socket) with a closed descriptor fails on the sending
    side with an OSError instead of leaving the peer waiting."""
    from triton_distributed_b200.runtime import fd_exchange as FX

    a, b = socket.socketpair(socket.AF_UNIX, socket.SOCK_STREAM)
    r, w = os.pipe()
    os.close(r)
    os.close(w)
    try:
        with pytest.raises(OSError):
            FX._send_fds(a, [r])
    finally:
        a.close()
        b.close()


def test_descriptor_exchange_round_trip_single_process():
    from triton_distributed_b200.runtime import fd_exchange as FX

    a, b = socket.socketpair(socket.AF_UNIX, socket.SOCK_STREAM)
    r, w = os.pipe()
    try:
        FX._send_fds(a, [r, w])
        got = FX._recv_fds(b, 2)
        assert len(got) == 2
        os.write(got[1], b"ping")
        assert os.read(r, 4) == b"ping"
        FX.close_fds(got)
    finally:
        for fd in (r, w):
            os.close(fd)
        a.close()
        b.close()


def test_heap_setup_keeps_ranks_in_step_when_one_rank_cannot_map():
    """A failure after the first agreement (exchange / import / map) on one rank: every rank runs the same
    collectives, all give the segment up, and each releases its handles and address range."""
    res, out = run_workers("heap_agreement_worker.py", 2, env={"CUDA_VISIBLE_DEVICES": ""}, timeout=120)
    assert res is not None, out[-2000:]
    assert all(r["none"] for r in res), res
    assert res[0]["calls"] == res[1]["calls"] and res[0]["calls"], res
    assert "map" in res[1]["err"] and "another rank" in res[0]["err"], res
    for r in res:
        assert r["released"] == 2 and r["freed"] == 1, res      # own + imported handle, the reserved range
    assert res[0]["unmapped"] == 2 and res[1]["unmapped"] == 0, res
