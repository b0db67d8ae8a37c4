"""Each device primitive through its own kernel, ranks emulated on one GPU (send halves first, then
the waiting halves). Follows the reference's test_notify.py, test_ring_put.py, test_nvshmem_api.py and
test_common_ops.py (grid barrier over random grid sizes)."""
import random

import pytest
import torch

from triton_distributed_b200.ops import primitives as P
from triton_distributed_b200.runtime import LocalWorld, check_status

pytestmark = pytest.mark.gpu


@pytest.fixture
def ring(cuda_device):
    world = 4
    lw = LocalWorld(world, cuda_device)
    ctxs = [P.create_primitive_context(r, world, 4096, heap=lw.heap(r)) for r in range(world)]
    for c in ctxs:
        c.source.copy_(torch.randint(0, 256, (c.nbytes,), dtype=torch.uint8, device=cuda_device))
    return ctxs


def _both_phases(ctxs, op, **kw):
    for c in ctxs:
        P.run_primitive(c, op, phase=1, **kw)
    for c in ctxs:
        P.run_primitive(c, op, phase=2, **kw)
    check_status()


def test_ring_put_int_p(ring):
    _both_phases(ring, "ring_put")
    for r, c in enumerate(ring):
        assert int(c.slot(0).view(torch.int32)[0]) == (r - 1) % len(ring) + 100


def test_notify_wait_ring_and_consume_token(ring):
    for value in (5, 6):  # two rounds: signals are plain values, no reset in between
        _both_phases(ring, "notify_wait", value=value)
        for r, c in enumerate(ring):
            assert c.result[:2].tolist() == [1, (r - 1) % len(ring) + 7]


def test_notify_add_to_rank0(ring):
    _both_phases(ring, "notify_add", value=len(ring))
    assert int(ring[0].result[0]) == 1 and int(ring[0].sig.local[1]) == len(ring)


@pytest.mark.parametrize("scope", ["thread", "warp", "block"])
def test_putmem_signal_scopes(ring, scope):
    _both_phases(ring, "put_signal", value=42, scope=scope)
    for r, c in enumerate(ring):
        prev = (r - 1) % len(ring)
        assert int(c.result[0]) == 1
        assert torch.equal(c.slot(prev), ring[prev].source)


def test_put_quiet_signal_add_and_get(ring):
    _both_phases(ring, "put_quiet_signal", value=3)
    for r, c in enumerate(ring):
        prev = (r - 1) % len(ring)
        assert int(c.result[0]) == 1 and torch.equal(c.slot(prev), ring[prev].source)
        c.slot(prev).zero_()
    _both_phases(ring, "get")
    for r, c in enumerate(ring):
        prev = (r - 1) % len(ring)
        assert torch.equal(c.slot(prev), ring[prev].source)


@pytest.mark.parametrize("scope", ["thread", "warp", "block"])
def test_broadcast_and_fcollect(ring, scope):
    """broadcast / fcollect at thread, warp and block scope (the thread and warp forms are what a kernel calls from a
    single lane or warp of a busy CTA)."""
    _both_phases(ring, "broadcast", scope=scope)
    for c in ring:
        assert torch.equal(c.slot(0), ring[0].source)
    for c in ring:
        for s in range(len(ring)):
            c.slot(s).zero_()
    _both_phases(ring, "fcollect", scope=scope)
    for c in ring:
        for s in range(len(ring)):
            assert torch.equal(c.slot(s), ring[s].source)


@pytest.mark.parametrize("scope", ["thread", "warp"])
def test_getmem_nbi_thread_and_warp_scope(ring, scope):
    for c in ring:
        for s in range(len(ring)):
            c.slot(s).zero_()
    _both_phases(ring, "get", scope=scope)
    for r, c in enumerate(ring):
        prev = (r - 1) % len(ring)
        assert torch.equal(c.slot(prev), ring[prev].source)


@pytest.mark.parametrize("scope", ["thread", "warp", "block"])
def test_barrier_all_scopes_single_rank(cuda_device, scope):
    """barrier_all / barrier_all_warp / barrier_all_block over 200 rounds on a one-rank world (ranks of one GPU must
    not wait for each other across launches): every round publishes the next epoch into this rank's own flag word
    and waits for it; the epoch counter must have advanced by exactly the number of rounds and no wait may fail."""
    lw = LocalWorld(1, cuda_device)
    ctx = P.create_primitive_context(0, 1, 256, heap=lw.heap(0))
    P.run_primitive(ctx, "barrier", value=200, scope=scope)
    check_status()
    assert int(ctx.result[0]) == 0
    assert int(ctx.barrier_epoch[0]) == 200 and int(ctx.sig.local[8]) == 200


def test_grid_barrier_random_grids(cuda_device):
    lw = LocalWorld(1, cuda_device)
    ctx = P.create_primitive_context(0, 1, 4096, heap=lw.heap(0))
    rng = random.Random(0)
    for it in range(50):
        P.run_primitive(ctx, "grid_barrier", value=it * 1000, grid=rng.randint(1, 148))
    check_status()
    assert int(ctx.result[0]) == 0  # no CTA saw a stale neighbour


def test_host_stream_ops_put_signal_wait(cuda_device):
    """pynvshmem-style host API on emulated ranks of one GPU: rank 0 puts a block into rank 1 and raises a
    signal in stream order; rank 1's stream-ordered wait passes; a wait on a word nothing sets runs out and
    reports instead of blocking the stream for good."""
    import torch
    from triton_distributed_b200 import _lib
    from triton_distributed_b200.runtime import LocalWorld, check_status, shmem_host as SH

    lw = LocalWorld(2, cuda_device)
    data = [lw.heap(r).zeros((4096,), torch.float32) for r in range(2)]
    sig = [lw.heap(r).zeros((8,), torch.int64) for r in range(2)]
    src = torch.arange(4096, device=cuda_device, dtype=torch.float32)
    SH.putmem_signal_on_stream(data[0], src, sig[0], 3, 5, SH.NVSHMEM_SIGNAL_SET, pe=1)
    SH.signal_op_on_stream(sig[0], 3, 2, SH.NVSHMEM_SIGNAL_ADD, pe=1)
    SH.signal_wait_until_on_stream(sig[1], 3, SH.NVSHMEM_CMP_EQ, 7)
    torch.cuda.synchronize()
    check_status()
    assert torch.equal(data[1].local, src) and int(sig[1].local[3]) == 7
    got = torch.empty_like(src)
    SH.getmem_on_stream(got, data[0], pe=1)
    torch.cuda.synchronize()
    assert torch.equal(got, src)
    # a flag that nothing sets: the wait gives up after its limit (0.2 s here) and says so
    from triton_distributed_b200.runtime import global_status
    _lib.check(_lib.lib().tdist_signal_wait_on_stream(sig[1].local.data_ptr() + 8 * 5, SH.NVSHMEM_CMP_GE, 1, global_status().device_ptr,
                                                      200_000_000, torch.cuda.current_stream().cuda_stream), "wait")
    torch.cuda.synchronize()
    with pytest.raises(_lib.TdistTimeoutError):
        check_status()
    torch.cuda.synchronize()
    check_status()  # the record was cleared and the context still works


@pytest.mark.parametrize("grid", [1, 7, 64])
def test_scoped_loads_stores_atomics_and_warp_intrinsics(cuda_device, grid):
    """red / atom / CAS at gpu and sys scope, release-acquire hand-over and the warp intrinsics, counted exactly
    (the reference's test_language_extra.py checks the same helpers through Triton kernels)."""
    lw = LocalWorld(1, cuda_device)
    ctx = P.create_primitive_context(0, 1, 4096, heap=lw.heap(0))
    ctx.slot(0).zero_()
    ctx.result.zero_()
    P.run_primitive(ctx, "scoped_ops", grid=grid)
    torch.cuda.synchronize()
    check_status()
    w = ctx.slot(0).view(torch.int32)[:6].tolist()
    threads = grid * 256
    assert int(ctx.result[0]) == 0
    assert w[0] == threads and w[1] == threads and w[2] == 0 and w[3] == grid and w[5] == threads // 32
