"""Planning entry points of the C ABI that need no GPU: fusion discovery (the reference's known answers through
the library, not through Python), the shard plan, the code generator's answer, the reference-named FFI alias, the
tuning options, and the struct sizes the binding checks at load."""
import ctypes
import json

import pytest

from symplex_b200 import _capi, fusion, sharding


def _discover(lib, ops):
    arr, _keep = _capi.pack_fusion_ops(ops)
    buf = ctypes.create_string_buffer(8192)
    n = lib.symplex_b200_discover_fusions(arr, len(ops), buf, 8192)
    assert n == len(buf.value)
    return buf.value.decode()


def test_reference_kat_matmul_bias_relu_through_the_c_abi(lib):
    # rust-engine/src/fusion_engine.rs:2469-2483 and :2558-2573
    ops = [("matmul", [128, 256], "fp16"), ("add", [128, 256], "fp16"), ("relu", [128, 256], "fp16")]
    text = _discover(lib, ops)
    d = json.loads(text)
    assert len(d["boundaries"]) == 1
    b = d["boundaries"][0]
    assert b["pattern"] == "MatMulBiasReLU" and b["op_indices"] == [0, 1, 2]
    assert b["memory_traffic_savings_bytes"] == 2 * 65536 + 2 * 65536 == d["total_hbm_traffic_reduction"]
    assert d["requires_polyhedral_validation"] is True
    # compute_confidence: 0.9 + 0.1 (one rank) + 0.05 (one dtype) + 0.05 (not in place), clamped to 1
    assert b["confidence"] == 1.0 and b["compute_savings_factor"] == 1.1
    # estimated_speedup: 1.1 * (1 + mb / (mb + 10)) * confidence with mb = 0.25
    assert d["total_estimated_speedup"] == pytest.approx(1.1 * (1 + 0.25 / 10.25), abs=6e-4)
    # the reference's formatting: three decimals for the total, two for the per-boundary factors
    assert '"total_estimated_speedup": 1.127,' in text and '"compute_savings_factor": 1.10, "confidence": 1.00}' in text


def test_no_boundary_for_a_single_op_or_a_foreign_chain(lib):
    # rust-engine/src/fusion_engine.rs:2534-2542: one op -> no boundary, speedup 1.0
    d = json.loads(_discover(lib, [("relu", [128], "fp32")]))
    assert d["boundaries"] == [] and d["total_estimated_speedup"] == 1.0 and d["requires_polyhedral_validation"] is False
    d = json.loads(_discover(lib, [("matmul", [8, 8], "bf16"), ("softmax", [8, 8], "bf16"), ("matmul", [8, 8], "bf16"),
                                   ("add", [8], "fp32")]))
    assert [b["op_indices"] for b in d["boundaries"]] == [[2, 3]]
    assert d["boundaries"][0]["confidence"] == 0.95  # ranks differ, dtypes differ: 0.9 + 0.05
    assert json.loads(_discover(lib, []))["boundaries"] == []


def test_buffer_too_small_reports_the_needed_size(lib):
    ops = [("matmul", [4, 4], "fp32"), ("gelu", [4, 4], "fp32")]
    arr, _keep = _capi.pack_fusion_ops(ops)
    small = ctypes.create_string_buffer(16)
    need = lib.symplex_b200_discover_fusions(arr, 2, small, 16)
    assert need < -100 and small.value == b""
    big = ctypes.create_string_buffer(-need)
    assert lib.symplex_b200_discover_fusions(arr, 2, big, -need) == -need - 1


def test_python_module_is_a_face_of_the_library(lib):
    ops = [("matmul", [64, 64], "bf16"), ("mul", [64, 64], "bf16"), ("add", [64, 64], "bf16"), ("silu", [64, 64], "bf16")]
    assert fusion.discover_fusions(ops) == _discover(lib, ops)
    d = _capi.GemmDesc()
    ep = fusion.compile_epilogue(["matmul", "mul", "add", "silu"], d)
    assert (ep.activation, ep.has_bias, ep.has_scale, ep.consumed) == ("silu", True, True, 4) and d.activation == _capi.ACT_SILU


def test_compile_epilogue_from_the_middle_of_a_list(lib):
    ops = [("relu", [8], "fp32"), ("matmul", [8, 8], "fp32"), ("add", [8, 8], "fp32"), ("tanh", [8, 8], "fp32"),
           ("exp", [8, 8], "fp32")]
    arr, _keep = _capi.pack_fusion_ops(ops)
    d = _capi.GemmDesc()
    c, b, s = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    f = lib.symplex_b200_compile_epilogue
    assert f(arr, 5, 1, ctypes.byref(d), ctypes.byref(c), ctypes.byref(b), ctypes.byref(s)) == 0
    assert (c.value, b.value, s.value, d.activation) == (3, 1, 0, _capi.ACT_TANH)
    assert f(arr, 5, 0, ctypes.byref(d), ctypes.byref(c), ctypes.byref(b), ctypes.byref(s)) == _capi.ERR_INVALID
    assert f(arr, 5, 5, ctypes.byref(d), ctypes.byref(c), ctypes.byref(b), ctypes.byref(s)) == _capi.ERR_INVALID


@pytest.mark.parametrize("M,N,K,world", [(65536, 8192, 8192, 8), (1024, 512, 256, 2), (768, 64, 32, 1)])
def test_shard_plan_pod_agrees_with_the_python_plan(lib, M, N, K, world):
    pod = _capi.ShardPlanPOD()
    assert lib.symplex_b200_analyze_matmul(M, N, K, world, 2, ctypes.byref(pod)) == 0
    plan = sharding.analyze_matmul(M, N, K, world)
    a, b, c = plan.tensor_shards
    assert pod.a.strategy == a.strategy.value == 1 and list(pod.a.local_shape) == a.local_shape == [M // world, K]
    assert pod.b.strategy == b.strategy.value == 0 and pod.b.shard_dim == -1 and list(pod.b.local_shape) == [K, N]
    assert pod.c.strategy == c.strategy.value == 1 and list(pod.c.original_shape) == [M, N]
    assert pod.total_communication_bytes == plan.total_communication_bytes
    assert pod.peak_memory_per_device == plan.peak_memory_per_device
    assert pod.n_all_gather_ops == len(plan.all_gather_ops) == (1 if world > 1 else 0)
    assert pod.n_all_reduce_ops == 0 and pod.n_all_to_all_ops == 0 and pod.world == world


def test_shard_plan_rejects_an_uneven_split(lib):
    pod = _capi.ShardPlanPOD()
    assert lib.symplex_b200_analyze_matmul(1000, 8, 8, 3, 2, ctypes.byref(pod)) == _capi.ERR_INVALID
    assert lib.symplex_b200_analyze_matmul(1024, 8, 8, 0, 2, ctypes.byref(pod)) == _capi.ERR_INVALID


def test_reference_named_micro_kernel_config_symbol(lib):
    # rust-engine/tests/integration.rs:11-17: ServerX86, 4-byte elements -> an 8 x 8 tile
    out = [ctypes.c_size_t() for _ in range(5)]
    lib.poly_get_micro_kernel_config(0, 4, *[ctypes.byref(o) for o in out])
    assert (out[0].value, out[1].value) == (8, 8)
    mine = [ctypes.c_size_t() for _ in range(5)]
    for target, eb in [(0, 4), (0, 2), (1, 4), (2, 4), (3, 2), (3, 4)]:
        lib.poly_get_micro_kernel_config(target, eb, *[ctypes.byref(o) for o in out])
        lib.symplex_b200_micro_kernel_config(target, eb, *[ctypes.byref(o) for o in mine])
        assert [o.value for o in out] == [o.value for o in mine]
    lib.poly_get_micro_kernel_config(3, 2, None, None, None, None, None)  # null outputs are skipped


def test_generate_matmul_describes_the_dispatched_kernel(lib):
    gk = _capi.GeneratedKernel()
    assert lib.symplex_b200_generate_matmul(8192, 8192, 8192, 2, 128, 128, 32, ctypes.byref(gk)) == 0
    plan = _capi.GemmPlan()
    d = _capi.GemmDesc()
    lib.symplex_b200_gemm_desc_init(ctypes.byref(d), 8192, 8192, 8192, _capi.DT_BF16, _capi.DT_BF16)
    d.tile_n = 128
    assert lib.symplex_b200_gemm_plan(ctypes.byref(d), 0, ctypes.byref(plan)) == 0
    assert gk.valid == 1 and gk.kernel_name == plan.kernel_name
    assert list(gk.grid_dims) == list(plan.grid_dims) and list(gk.block_dims) == list(plan.block_dims)
    assert gk.shared_mem_bytes == plan.shared_mem_bytes
    assert 64 <= gk.register_count <= 255 and gk.register_count * gk.block_dims[0] <= 65536
    assert lib.symplex_b200_generate_matmul(512, 512, 512, 4, 0, 0, 0, ctypes.byref(gk)) == 0 and gk.valid == 1
    assert lib.symplex_b200_generate_matmul(0, 8, 8, 2, 0, 0, 0, ctypes.byref(gk)) == _capi.ERR_INVALID
    assert gk.valid == 0 and gk.error_message
    assert lib.symplex_b200_generate_matmul(8, 8, 8, 8, 0, 0, 0, ctypes.byref(gk)) == _capi.ERR_INVALID


def test_options_round_trip_and_change_the_plan(lib):
    assert lib.symplex_b200_get_option(b"no_such_option") == -2 ** 63
    assert lib.symplex_b200_set_option(b"no_such_option", 1) == _capi.ERR_INVALID
    assert lib.symplex_b200_get_option(b"pair_mode") == -1 and lib.symplex_b200_get_option(b"wait_limit_ms") == 2000
    d = _capi.GemmDesc()
    lib.symplex_b200_gemm_desc_init(ctypes.byref(d), 8192, 8192, 8192, _capi.DT_BF16, _capi.DT_BF16)
    plan = _capi.GemmPlan()
    lib.symplex_b200_gemm_plan(ctypes.byref(d), 148, ctypes.byref(plan))
    assert (plan.tile_m, plan.cluster_size) == (512, 2)
    with _capi.option("pair_mode", 0):
        assert lib.symplex_b200_get_option(b"pair_mode") == 0
        lib.symplex_b200_gemm_plan(ctypes.byref(d), 148, ctypes.byref(plan))
        assert (plan.tile_m, plan.cluster_size) == (128, 1)
    assert lib.symplex_b200_get_option(b"pair_mode") == -1


def test_abi_sizes_cover_every_struct(lib):
    n = lib.symplex_b200_abi_sizes_ext(None, 0)
    assert n == 10
    sizes = (ctypes.c_int32 * n)()
    lib.symplex_b200_abi_sizes_ext(sizes, n)
    assert list(sizes)[5:] == [ctypes.sizeof(t) for t in (_capi.Comm, _capi.ShardPlanPOD, _capi.GeneratedKernel,
                                                           _capi.FusionOp, _capi.KernelArgs)]
    first = (ctypes.c_int32 * 5)()
    lib.symplex_b200_abi_sizes(ctypes.byref(first))
    assert list(first) == list(sizes)[:5]


def test_sharded_gemm_argument_checks_without_a_gpu(lib):
    d = _capi.GemmDesc()
    lib.symplex_b200_gemm_desc_init(ctypes.byref(d), 1024, 64, 64, _capi.DT_BF16, _capi.DT_BF16)
    comm = _capi.Comm()
    buf = (ctypes.c_float * 16)()
    f = lib.symplex_b200_sharded_gemm
    assert f(ctypes.byref(d), buf, buf, None, None, 0, None) == _capi.ERR_INVALID
    comm.rank, comm.world = 0, 9
    assert f(ctypes.byref(d), buf, buf, None, ctypes.byref(comm), 0, None) == _capi.ERR_INVALID
    comm.world = 3  # 1024 rows do not split over 3 ranks
    assert f(ctypes.byref(d), buf, buf, None, ctypes.byref(comm), 0, None) == _capi.ERR_INVALID
    comm.world = 2
    assert f(ctypes.byref(d), buf, buf, None, ctypes.byref(comm), 7, None) == _capi.ERR_INVALID  # unknown exchange
    assert f(ctypes.byref(d), buf, buf, None, ctypes.byref(comm), 0, None) == _capi.ERR_INVALID  # no local C
    assert comm.epoch == 0, "a rejected call must not count as a collective call"
