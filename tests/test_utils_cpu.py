"""Host utilities that need no GPU: autotuner protocol, verbose comparison, data generation, trace
merging, and the torch restatements the CPU paths of the ops rely on."""
import pytest
import torch

import triton_distributed_b200.utils as U
from triton_distributed_b200.ops import flash_decode as FD
from triton_distributed_b200.ops import moe_utils as MU
from triton_distributed_b200.utils.autotuner import ContextualAutoTuner
from triton_distributed_b200.utils.profile import merge_traces


def test_contextual_autotune_picks_the_fastest_config(monkeypatch, tmp_path):
    monkeypatch.chdir(tmp_path)
    cost = {1: 3.0, 2: 1.0, 3: 2.0}
    seen = []

    @U.tunable(configs=[{"x": 1}, {"x": 2}, {"x": 3}], key=lambda n: n)
    def op(n, *, config):
        seen.append(config["x"])
        return n * config["x"]

    monkeypatch.setattr(ContextualAutoTuner, "timer", staticmethod(lambda fn: (lambda r: (r, cost[seen[-1]]))(fn())))

    @U.contextual_autotune(n_repeat=2, n_warmup=1)
    def step():
        return op(5) + op(7)

    assert step() == 5 * 2 + 7 * 2
    assert op.cache == {5: {"x": 2}, 7: {"x": 2}}
    # each config of each key was measured warmup + repeat times, one measurement per thunk run
    assert seen.count(1) == seen.count(3) == 2 * 3
    assert (tmp_path / ".autotune_logs" / "rank-0.log").read_text().count("best-config-id: 1") == 2
    n = len(seen)
    step()
    assert len(seen) == n + 2  # tuned: no more measuring


def test_assert_allclose_reports_where(capsys):
    a = torch.zeros(4, 4)
    b = a.clone()
    b[2, 3] = 1.0
    U.assert_allclose(a, a)
    with pytest.raises(AssertionError) as e:
        U.assert_allclose(a, b, atol=1e-3)
    assert "1 of 16" in str(e.value) and "(2, 3)" in str(e.value)


def test_generate_data_shapes_and_ranges():
    gen = U.generate_data([((3, 4), torch.float32, (2.0, 1.0)), ((5,), torch.int32, (3, 0))], device="cpu")
    x, y = next(gen)
    assert x.shape == (3, 4) and y.dtype == torch.int32
    assert x.min() >= -1.0 and x.max() <= 3.0 and y.abs().max() <= 3
    x2, _ = next(gen)
    assert not torch.equal(x, x2)


def test_merge_traces_separates_ranks():
    t0 = {"traceEvents": [{"pid": 7, "tid": 1, "name": "k", "ph": "X"}], "schemaVersion": 1}
    t1 = {"traceEvents": [{"pid": 7, "tid": 1, "name": "k", "ph": "X"}]}
    merged = merge_traces([t0, t1])
    pids = sorted(e["pid"] for e in merged["traceEvents"])
    assert pids == [7, 100_000_007] and merged["schemaVersion"] == 1


def test_cpu_restatements_agree_with_each_other():
    torch.manual_seed(0)
    ids = torch.randint(0, 6, (40, 3), dtype=torch.int32)
    r = MU.route(ids, 6)
    flat = ids.reshape(-1)
    assert torch.equal(flat[(r.sorted_token.long() * 0 + torch.argsort(r.slot_of.long()))], torch.sort(flat, stable=True).values)
    assert int(r.cumsum[-1]) == flat.numel()
    # lse merge of one part is the identity
    part = torch.cat([torch.randn(2, 3, 8), torch.randn(2, 3, 1)], -1)
    torch.testing.assert_close(FD.ref_lse_merge(part.unsqueeze(0)), part[..., :-1])


def test_parallel_strategies_on_cpu():
    """The strategy layer on one CPU process: column/row parallel linears (bf16-free fp32 path and the fp8
    path), sequence sharding arithmetic, expert placement."""
    import torch
    from triton_distributed_b200 import parallel as P

    st = P.init_parallel_state()
    assert st.world == 1 and st.is_single_node and st.nnodes == 1
    g = torch.Generator().manual_seed(0)
    w, x = torch.randn(64, 256, generator=g), torch.randn(8, 256, generator=g)
    torch.testing.assert_close(P.ColumnParallelLinear(w, 64, st)(x), x @ w.t(), rtol=1e-4, atol=1e-4)
    w2 = torch.randn(128, 256, generator=g)
    torch.testing.assert_close(P.RowParallelLinear(w2, 64, st)(x), x @ w2.t(), rtol=1e-4, atol=1e-4)
    y8 = P.ColumnParallelLinear(w, 64, st, fp8=True)(x).float()
    assert (y8 - x @ w.t()).abs().max() < 0.1 * (x @ w.t()).abs().max()
    lens = torch.tensor([10, 100, 3, 0])
    per_rank = P.kv_lens_per_rank(lens, 4)
    assert per_rank.shape == (4, 4) and torch.equal(per_rank.sum(0), lens.to(torch.int32))
    assert per_rank[:, 1].tolist() == [25, 25, 25, 25] and per_rank[:, 0].tolist() == [3, 3, 3, 1]
    kv = P.SequenceParallelKVCache.allocate(2, 100, 2, 8, 1, 4, device="cpu", dtype=torch.float32)
    assert kv.write(0, torch.ones(2, 8), torch.ones(2, 8), 30, 100) and not kv.write(0, torch.ones(2, 8), torch.ones(2, 8), 3, 100)
    ep = P.ExpertPlacement(8, 4)
    assert ep.owner(torch.tensor([0, 3, 7])).tolist() == [0, 1, 3]
    assert ep.send_counts(torch.tensor([[0, 3], [7, 7]])).tolist() == [[1, 0], [0, 1], [0, 0], [0, 2]]
    assert list(P.experts_of_rank(8, 2, 4)) == [4, 5]
    assert P.shard_rows(torch.arange(8).view(4, 2), 1, 2).tolist() == [[4, 5], [6, 7]]
    assert P.shard_columns(torch.arange(8).view(2, 4), 1, 2).tolist() == [[2, 3], [6, 7]]


def test_reference_names_resolve_on_cpu():
    """Names the reference exports that map onto the single-level paths here."""
    import torch
    from triton_distributed_b200.ops import collectives as CO, flash_decode as FD, gemm as G, moe_tp as MT, moe_utils as MU

    x = torch.randn(8, 4)
    assert CO.add_continuous(x, x).allclose(2 * x) and CO.copy_continuous(x, torch.empty_like(x)).equal(x)
    out = torch.empty(2, 4)
    assert CO.ring_reduce(x, out, 1, 4).allclose(x.view(4, 2, 4).sum(0))
    assert CO.inter_node_allgather is CO.cp_engine_producer_all_gather_intra_node
    assert G.ag_gemm_inter_node is G.ag_gemm_intra_node and MT.ag_group_gemm_inter_node is MT.ag_group_gemm_intra_node
    assert callable(FD.gqa_fwd_batch_decode_aot) and FD.gqa_fwd_batch_decode_persistent is FD.gqa_fwd_batch_decode
    padded = G.padded_to_BLOCK_M(torch.arange(12.0).view(6, 2), 2, 4)
    assert padded.shape == (8, 2) and padded[3].abs().sum() == 0 and padded[4].tolist() == [6.0, 7.0]
    ids = torch.tensor([[0, 3], [3, 1]], dtype=torch.int32)
    assert MU.bincount(ids, 4).tolist() == [1, 1, 0, 2]
    gather, scatter = MU.calc_gather_index(ids, 4)
    assert gather.tolist() == [0, 1, 0, 1] and scatter.tolist() == [0, 2, 3, 1]
    a, w = torch.randn(4, 8), torch.randn(6, 8)
    ctx = G.create_ag_gemm_inter_node_context(a, w, 0, 1)
    assert G.ag_gemm_inter_node(a, w, ctx).shape == (4, 6)
    rs = G.create_gemm_rs_context(4, 6, 0, 1, output_dtype=torch.float32, device="cpu")
    assert G.gemm_rs_op(a, w, rs).shape == (4, 6)


def test_config_catalogue_and_nvtx_decorator(monkeypatch):
    from triton_distributed_b200.utils import Config, nvtx_range

    c = Config.from_env({"TDIST_NVLS": "1", "TDIST_WAIT_TIMEOUT_MS": "250", "TDIST_GEMM_CTA_PAIR": "0", "TDIST_HEAP_BACKEND": "ipc"})
    assert c.nvls is True and c.wait_timeout_ms == 250.0 and c.gemm_cta_pair == 0 and c.heap_backend == "ipc"
    assert Config.from_env({}) == Config()
    text = c.describe()
    assert "TDIST_WAIT_TIMEOUT_MS" in text and "(default 4000.0)" in text and len(text.splitlines()) == len(Config.env_names())

    def f(x):
        return x + 1
    monkeypatch.delenv("TDIST_NVTX", raising=False)
    assert nvtx_range("t")(f) is f                      # off: the function is returned untouched
    monkeypatch.setenv("TDIST_NVTX", "1")
    g = nvtx_range("t")(f)
    assert g is not f and g(1) == 2 and g.__name__ == "f"  # on: wrapped; without CUDA the range calls are skipped


def test_top_level_namespace_and_remaining_reference_names():
    """`import triton_distributed_b200 as tdist` exposes the reference's public names; the EP helper functions and the
    pynvshmem-style host names exist and behave on CPU."""
    import torch
    import triton_distributed_b200 as tdist
    from triton_distributed_b200.ops import collectives as CO, flash_decode as FD
    from triton_distributed_b200.runtime import shmem_host as SH
    from triton_distributed_b200.utils import aot_compile_spaces, aot_spaces, get_triton_combine_kv_algo_info, p2p_native_atomic_required

    for name in ("ag_gemm_intra_node", "gemm_rs", "fast_allgather", "fast_all_to_all", "moe_dispatch", "gqa_fwd_batch_decode",
                 "sp_gqa_fwd_batch_decode", "ag_group_gemm_intra_node", "moe_reduce_rs", "select_experts", "AllGatherLayer",
                 "EPAll2AllLayer", "SpGQAFlashDecodeAttention", "initialize_distributed", "nvshmem_create_tensor",
                 "contextual_autotune", "group_profile", "nvls_allreduce", "ag_gemm_fp8"):
        assert hasattr(tdist, name), name
    recv_splits, recv_offset, n = tdist.get_ag_splits_and_recv_offset_for_dispatch(torch.tensor([3, 0, 2, 1], dtype=torch.int32), 1, 4)
    assert recv_splits.tolist() == [[3, 0, 2, 1]] and recv_offset.view(-1).tolist() == [0, 3, 3, 5] and n == 6
    reqs = tdist.get_dispatch_send_reqs_for_target_node(torch.tensor([0, 0, 1, 0, 0, 0, 1]), 0)
    assert reqs.tolist() == [[0, 2], [3, 6]]
    assert tdist.get_dispatch_send_reqs_for_target_node(torch.tensor([1, 1]), 0).shape == (0, 2)
    assert SH.nvshmem_my_pe() == 0 and SH.nvshmem_n_pes() == 1 and SH.nvshmem_team_n_pes(SH.NVSHMEMX_TEAM_NODE) == 1
    assert SH.NVSHMEM_SIGNAL_SET == 9 and SH.NVSHMEM_SIGNAL_ADD == 10 and SH.NVSHMEM_CMP_GE == 5
    assert CO.reduce_scatter_ring_push_1d_intra_node_sm is CO.reduce_scatter_ring_push_1d_intra_node_kernel
    assert FD.kernel_inter_rank_gqa_fwd_batch_decode_combine_kv is FD.inter_rank_combine
    assert get_triton_combine_kv_algo_info(32, 128)["BLOCK_DV"] == 128

    @aot_compile_spaces({"decode_bf16_d128": {"signature": "*bf16, *bf16, i32", "grid": ["B", "Hkv", "splits"]}})
    def kernel():
        return 7
    assert kernel() == 7 and aot_spaces()["decode_bf16_d128"]["function"] == "kernel"
    assert p2p_native_atomic_required(lambda: 5)() == 5


def test_bench_reference_arm_reports_unavailable():
    """`bench.py --impl reference` must print one JSON line and exit 0 even without a GPU: the reference cannot be
    installed offline, and the line says so."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, timeout=120, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stderr[-1000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and len(line["unavailable"]) > 10


@pytest.mark.parametrize("wide", [0, 1])
def test_gemm_static_schedule_gives_every_tile_to_one_unit(wide):
    """The kernel's tile schedule replayed on the host (the same function the device runs): every 256-column tile exactly
    once, for even and odd tile counts, full and partial last rounds, with and without the split first round."""
    import ctypes as C
    import random

    from triton_distributed_b200 import _lib
    lib = _lib.lib()
    rng = random.Random(3)
    span, first = C.c_int(0), C.c_int(0)
    cases = [(70, 8, 4, 24, 22), (70, 8, 4, 24, 0), (74, 1, 32, 24, 0), (69, 4, 8, 23, 0), (69, 4, 8, 23, 5)]
    for _ in range(300):
        units, world = rng.randint(1, 74), rng.randint(1, 8)
        seg_m, n_tiles = rng.randint(1, 9), rng.randint(1, 25)
        own = seg_m * ((n_tiles + 1) // 2)
        split = units - own if (wide and world > 1 and own < units and units - own <= own and rng.random() < 0.7) else 0
        cases.append((units, world, seg_m, n_tiles, split))
    for (units, world, seg_m, n_tiles, split) in cases:
        if not wide:
            split = 0
        for rank in {0, world - 1}:
            rc = lib.tdist_gemm_schedule_check(wide, units, world, rank, seg_m, n_tiles, rng.choice([0, 1, 4, 8]), split,
                                               C.byref(span), C.byref(first))
            assert rc == 0, (wide, units, world, rank, seg_m, n_tiles, split, rc)
            total = world * seg_m * n_tiles
            assert span.value * units >= total
            if split and n_tiles % 2 == 0:
                assert first.value >= 1     # nobody starts on a peer's segment (an odd last tile has no second half to give)


def test_gemm_split_first_round_balances_the_headline_problem():
    """m8192 n49152 k12288 at tp8 with 8 pusher CTAs: 70 CTA pairs, 48 own wide items, 384 in all. Cutting 22 own items in
    two keeps every unit busy with local rows for the first half item and all units end after 5.5 items."""
    import ctypes as C

    from triton_distributed_b200 import _lib
    lib = _lib.lib()
    span, first = C.c_int(0), C.c_int(0)
    assert lib.tdist_gemm_schedule_check(1, 70, 8, 3, 4, 24, 0, 22, C.byref(span), C.byref(first)) == 0
    assert span.value == 11 and first.value == 1
    assert lib.tdist_gemm_schedule_check(1, 70, 8, 3, 4, 24, 0, 0, C.byref(span), C.byref(first)) == 0
    assert span.value == 11 and first.value == 0


def test_ag_gemm_launch_plan_follows_the_measured_optima():
    """The pusher-count / tiling model of the fused AG-GEMM, on the shapes it was calibrated with: the long-K headline
    problem takes the wide tiling with 8 / 4 / 2 pusher CTAs at tp8 / tp4 / tp2 (8 x B200: 8 pushers 0.97 ms, 6 pushers
    1.19 ms, 10 pushers 1.02 ms); the all-gather-bound short-K problem takes 256 x 256 tiles and many pushers (4 x B200:
    16 pushers 158 us, 8 pushers 226 us)."""
    import ctypes as C

    from triton_distributed_b200 import _lib
    lib = _lib.lib()

    def plan(world, m, n, k):
        g = _lib.GemmArgs()
        g.mode, g.world, g.rank, g.m_per_rank, g.n, g.k, g.cta_pair = _lib.GEMM_AG, world, 0, m // world, n // world, k, -1
        out = (C.c_int * 4)()
        assert lib.tdist_gemm_plan(C.byref(g), out) == 0
        return list(out)

    if plan(8, 8192, 49152, 12288)[3] != 148:
        pytest.skip("calibrated for 148 SMs")
    assert plan(8, 8192, 49152, 12288)[:3] == [2, 1, 8]
    assert plan(4, 8192, 49152, 12288)[:3] == [2, 1, 4]
    assert plan(2, 8192, 49152, 12288)[:3] == [2, 1, 2]
    ctas, wide, pushers, _ = plan(4, 8192, 11008, 4096)
    assert (ctas, wide) == (2, 0) and 12 <= pushers <= 18
    ctas, wide, pushers, _ = plan(8, 8192, 11008, 4096)
    assert (ctas, wide) == (2, 0) and 14 <= pushers <= 18


def test_counters_are_cleared_once_after_a_reported_abort(monkeypatch):
    """Kernels that keep arrival counters in device memory leave them at zero; after a wait was reported (the launch
    was cut short) the next use of the buffer clears them again, and only that one."""
    from triton_distributed_b200.runtime import status as S

    class FakeStatus:
        aborts = 0

    fake = FakeStatus()
    monkeypatch.setattr(S, "global_status", lambda: fake)
    t = torch.arange(12, dtype=torch.int32)
    S.counters_clean(t, 8)
    assert t[8:].tolist() == [8, 9, 10, 11]          # nothing was reported: untouched
    fake.aborts = 1
    S.counters_clean(t, 8)
    assert t[:8].tolist() == list(range(8)) and t[8:].tolist() == [0, 0, 0, 0]
    t[8:] = 5
    S.counters_clean(t, 8)
    assert t[8:].tolist() == [5, 5, 5, 5]            # same generation: not again


def test_launch_heuristics_on_the_host():
    """Host-side choices that need no GPU: KV splits of flash decode (at least 256 keys per split, one wave of the machine
    at most), the flag words of a staged row gather, the push order of the MoE all-gather."""
    from triton_distributed_b200.ops import flash_decode as FD
    from triton_distributed_b200.ops import moe_tp as MT

    dev = torch.device("cpu")
    assert FD.default_splits(1, 8, 4096, dev) == 16          # 4096 keys -> 16 splits of 256
    assert FD.default_splits(1, 8, 100, dev) == 1
    assert FD.default_splits(8, 8, 131072, dev) <= 8         # 64 (batch, head) pairs already fill the machine
    assert 16 <= FD.default_splits(1, 8, 1 << 20, dev) <= 256
    flags = MT.staging_flags(1000, dev)                      # 8 blocks: 8 flags + 4 + 8 counters
    assert flags.dtype == torch.int32 and flags.numel() == 2 * 8 + 4 and int(flags.abs().sum()) == 0
    assert MT._ag_push_mode(2) == "push" and MT._ag_push_mode(4) == "push" and MT._ag_push_mode(8) == "push_ordered"


def test_every_name_of_the_reference_api_sheet_is_in_the_top_level_namespace():
    """A user of the reference finds its public Python names on ``import triton_distributed_b200 as tdist``: runtime and
    pynvshmem-style host calls, utilities, op contexts and ops, layers, decorators."""
    import math

    import triton_distributed_b200 as tdist
    names = """initialize_distributed TP_GROUP nvshmem_create_tensor nvshmem_create_tensor_list_intra_node symm_tensor
    nvshmem_barrier_all nvshmemx_barrier_all_on_stream nvshmem_my_pe nvshmem_n_pes nvshmem_team_my_pe nvshmem_team_n_pes
    nvshmem_ptr nvshmemx_mc_ptr nvshmemx_putmem_on_stream nvshmemx_putmem_signal_on_stream nvshmem_putmem nvshmem_getmem
    nvshmem_int_p wait_eq set_signal barrier_all_on_stream perf_func dist_print group_profile generate_data assert_allclose
    init_seed get_has_nvlink get_numa_world_size check_p2p_native_atomic_supported p2p_native_atomic_required
    create_ag_gemm_intra_node_context ag_gemm_intra_node gemm_persistent gemm_non_persistent create_ag_gemm_inter_node_context
    ag_gemm_inter_node create_gemm_rs_context gemm_rs create_reduce_scater_2d_ctx reduce_scatter_2d_op ring_reduce
    reduce_scatter_ring_push_1d_intra_node_ce reduce_scatter_ring_push_1d_intra_node_sm
    cp_engine_producer_all_gather_intra_node inter_node_allgather AllGatherMethod get_auto_all_gather_method
    create_fast_allgather_context fast_allgather AllGatherLayer create_all_to_all_context fast_all_to_all
    all_to_all_post_process EPAll2AllLayer bincount get_dispatch_send_reqs_for_target_node
    get_ag_splits_and_recv_offset_for_dispatch gqa_fwd_batch_decode gqa_fwd_batch_decode_intra_rank
    gqa_fwd_batch_decode_persistent gqa_fwd_batch_decode_aot gqa_fwd_batch_decode_intra_rank_aot
    gqa_fwd_batch_decode_persistent_aot get_triton_combine_kv_algo_info kernel_inter_rank_gqa_fwd_batch_decode_combine_kv
    SpGQAFlashDecodeAttention sort_topk_ids_align_block_size create_ag_group_gemm_intra_node_context
    ag_group_gemm_intra_node ag_group_gemm_inter_node create_ag_group_gemm_inter_node_context select_experts create_moe_rs_context moe_reduce_rs
    contextual_autotune aot_compile_spaces""".split()
    missing = [n for n in names if not hasattr(tdist, n)]
    assert not missing, missing

    # the *_aot variants are the same calls with the stream in front (None = current stream)
    torch.manual_seed(0)
    B, Hq, Hkv, D, page = 2, 4, 2, 64, 4
    q = torch.randn(B, Hq, D)
    k = torch.randn(6, page, Hkv, D)
    v = torch.randn(6, page, Hkv, D)
    lens = torch.tensor([5, 9], dtype=torch.int32)
    table = torch.tensor([[0, 1, 2], [3, 4, 5]], dtype=torch.int32)
    scale = 1.0 / math.sqrt(D)
    want = tdist.gqa_fwd_batch_decode(q, k, v, None, None, lens, table, scale)
    got = tdist.gqa_fwd_batch_decode_aot(None, q, k, v, None, None, lens, table, scale)
    assert torch.equal(got, want)
    part = tdist.gqa_fwd_batch_decode_intra_rank_aot(None, q, k, v, None, None, lens, table, scale)
    assert part.shape == (B, Hq, D + 1) and torch.allclose(part[..., :D], want, atol=1e-5)
    assert tdist.bincount(torch.tensor([[0, 2], [2, 1]], dtype=torch.int32), 4).tolist() == [1, 1, 2, 0]


def test_small_utilities_of_the_reference(tmp_path):
    """is_cuda / is_hip / is_fp8_dtype, the deterministic-mode guard, CUDA_CHECK, the tolerant trace loader and the
    nvidia-smi / sysfs topology parsers, all without a GPU."""
    import enum
    import json

    from triton_distributed_b200 import utils as U

    assert U.is_hip() is False and U.is_cuda() == (torch.cuda.is_available() and torch.version.hip is None)
    assert U.is_fp8_dtype(torch.float8_e4m3fn) and U.is_fp8_dtype(torch.float8_e5m2)
    assert not U.is_fp8_dtype(torch.int8) and not U.is_fp8_dtype(torch.bfloat16)

    before = torch.are_deterministic_algorithms_enabled()
    with pytest.raises(ValueError):
        with U.with_torch_deterministic(not before):
            assert torch.are_deterministic_algorithms_enabled() == (not before)
            raise ValueError("inside")
    assert torch.are_deterministic_algorithms_enabled() == before

    class Res(enum.IntEnum):
        OK = 0
        BAD = 700
    assert U.CUDA_CHECK(Res.OK) is None and U.CUDA_CHECK((Res.OK, 42)) == 42 and U.CUDA_CHECK((0, 1, 2)) == (1, 2)
    with pytest.raises(RuntimeError, match="700"):
        U.CUDA_CHECK((Res.BAD, None))

    good = tmp_path / "trace_rank3.json"
    good.write_text(json.dumps({"traceEvents": [{"ph": "M", "name": "process_name", "pid": 7, "args": {"name": "python"}},
                                                {"ph": "X", "name": "k", "pid": 7, "tid": 1, "ts": 0, "dur": 1}]}))
    ev = U.process_trace_json(str(good))
    assert ev[1]["pid"] == 7 + 3 * 100_000_000 and ev[0]["args"]["name"].startswith("rank 3")
    bad = tmp_path / "bad.json"
    bad.write_text('{"traceEvents": [{"ph": "X", "name": "void f<"a">(int)\x01", "pid": 1}]}')
    tr = U.load_json(str(bad))
    assert tr["traceEvents"][0]["pid"] == 1 and '"' not in tr["traceEvents"][0]["name"]

    topo = ("\tGPU0\tGPU1\tGPU2\tNIC0\tCPU Affinity\n"
            "GPU0\t X \tNV18\tNV18\tSYS\t0-55\n"
            "GPU1\tNV18\t X \tPIX\tSYS\t0-55\n"
            "GPU2\tNV18\tPIX\t X \tSYS\t56-111\n"
            "NIC0\tSYS\tSYS\tSYS\t X \n")
    assert U.NvidiaSmiUtil.parse_topo_matrix(topo) == [[0, 1, 1], [1, 0, -1], [1, -1, 0]]
    dev = tmp_path / "0000:17:00.0"
    dev.mkdir()
    (dev / "numa_node").write_text("1\n")
    assert U.NvidiaSmiUtil.numa_node_of_bus_id("00000000:17:00.0\n", str(tmp_path)) == 1
    assert U.NvidiaSmiUtil.numa_node_of_bus_id("00000000:99:00.0", str(tmp_path)) == -1
