"""Planning queries (host only): hardware target, micro-kernel configuration, kernel choice and launch geometry.
Known answers come from the reference's own tests: LaunchConfig::matmul(128, 64, 32, 32) -> grid (2, 4) and
LaunchConfig::elementwise(1024, 256) -> 4 blocks (rust-engine/src/cuda_backend.rs:1508-1519), and
configure_extreme_ml_kernel(ServerX86, 4) -> tile 8 x 8 (rust-engine/tests/integration.rs:11-17)."""
import pytest

from symplex_b200 import _capi, _symplex_core, planner


def test_launch_config_known_answers():
    cfg = planner.LaunchConfig.matmul(128, 64, 32, 32)
    assert cfg.grid[0] == 2 and cfg.grid[1] == 4 and cfg.block == (32, 1, 1)
    assert cfg.shared_mem_bytes == 32 * 32 * 4 * 2
    e = planner.LaunchConfig.elementwise(1024, 256)
    assert e.grid[0] == 4 and e.block[0] == 256 and e.shared_mem_bytes == 0
    assert planner.LaunchConfig.elementwise(1025, 256).grid[0] == 5


def test_micro_kernel_config_reference_table(lib):
    # rust-engine/src/polyhedral.rs:4375-4422
    assert planner.micro_kernel_config("server", "fp32") == {
        "tile_m": 8, "tile_n": 8, "tile_k": 8, "accumulator_registers": 16, "prefetch_distance": 1,
        "double_buffer_count": 2}
    assert planner.micro_kernel_config("server", "bf16") == {
        "tile_m": 16, "tile_n": 16, "tile_k": 32, "accumulator_registers": 8, "prefetch_distance": 2,
        "double_buffer_count": 2}
    t = planner.micro_kernel_config("tensor", "fp16")
    assert (t["tile_m"], t["tile_n"], t["tile_k"], t["prefetch_distance"]) == (16, 16, 16, 4)
    e = planner.micro_kernel_config("edge", "fp32")
    assert (e["tile_m"], e["tile_n"], e["tile_k"], e["accumulator_registers"], e["double_buffer_count"]) == (4, 4, 8, 4, 1)
    # unknown names fall back the way parse_target / parse_element_type do
    assert planner.micro_kernel_config("mainframe", "complex128") == planner.micro_kernel_config("server", "fp32")
    assert _symplex_core.micro_kernel_config() == planner.micro_kernel_config("server", "fp32")


def test_micro_kernel_config_b200(lib):
    b = planner.micro_kernel_config("b200", "bf16")
    assert (b["tile_m"], b["tile_n"], b["tile_k"]) == (128, 256, 16)      # one tcgen05.mma, kind::f16
    assert b["accumulator_registers"] == 512                                # tensor-memory columns
    assert b["double_buffer_count"] == b["prefetch_distance"] + 1 >= 3
    f = planner.micro_kernel_config("b200", "fp32")
    assert (f["tile_m"], f["tile_n"], f["tile_k"]) == (128, 128, 8)        # kind::tf32


def test_hardware_target(lib):
    t = planner.hardware_target()
    assert t["warp_size"] == 32 and t["max_threads_per_sm"] == 2048
    assert (t["mma_m"], t["mma_n"], t["mma_k"], t["mma_pair_m"], t["mma_dtype"]) == (128, 256, 16, 256, "bf16")
    assert t["max_shared_mem_per_block"] == 227 * 1024 and t["tensor_memory_bytes_per_sm"] == 256 * 1024
    assert t["has_tma"] == 1 and t["has_tensor_memory"] == 1
    assert t["global_bw_gbps"] < t["global_bw_nominal_gbps"] and t["bf16_dense_tflops"] < t["bf16_dense_tflops_nominal"]
    if not t["from_device"]:
        assert t["num_sms"] == 148


CONFIGS = [
    # name, args, kwargs, kernel, tile, cluster
    ("cfg1", (512, 512, 512), dict(dtype="fp32"), "gemm_f32_fused_kernel", (128, 64, 32), 4),  # split-K over a cluster
    ("cfg2_bf16", (4096, 4096, 4096), dict(dtype="bf16", out_dtype="fp32", b_layout=_capi.COL_MAJOR),
     "gemm_pair_kernel", (512, 256, 64), 2),  # 2 waves of 512x256 beat 4 waves of 256x256
    ("cfg2_fp32", (4096, 4096, 4096), dict(dtype="fp32", b_layout=_capi.COL_MAJOR), "gemm_tf32x3_kernel", (128, 128, 32), 1),
    ("cfg3", (8192, 16384, 4096), dict(dtype="bf16", activation="gelu"), "gemm_pair_kernel", (512, 256, 64), 2),
    ("cfg4", (64, 64, 64), dict(dtype="fp32", batch=2048), "gemm_f32_small_kernel", (64, 64, 32), 1),
    ("cfg5", (65536, 8192, 8192), dict(dtype="bf16"), "gemm_pair_kernel", (512, 256, 64), 2),
    ("small_bf16", (256, 192, 128), dict(dtype="bf16"), "gemm_tc_kernel", (128, 64, 64), 1),
]


@pytest.mark.parametrize("name,args,kwargs,kernel,tile,cluster", CONFIGS, ids=[c[0] for c in CONFIGS])
def test_compile_matmul_for_the_baseline_configs(lib, name, args, kwargs, kernel, tile, cluster):
    r = planner.compile_matmul(*args, num_sms=148, **kwargs)
    assert r.valid and r.error == ""
    assert r.kernel_name == kernel and r.optimal_tile == tile and r.cluster_size == cluster
    M, N, K = args
    batch = kwargs.get("batch", 1)
    if kernel == "gemm_f32_small_kernel":  # its unit of work holds two problems
        assert r.tiles == -(-N // tile[1]) * -(-batch // 2) and r.mma_shape == (128, 128, 8)
    else:
        assert r.tiles == -(-M // tile[0]) * -(-N // tile[1]) * batch
    assert 1 <= r.grid_dims[0] <= 148 and r.grid_dims[0] % cluster == 0 and r.grid_dims[1:] == (1, 1)
    assert r.block_dims[0] in (192, 320, 448) and r.shared_mem_bytes <= 227 * 1024 and r.tmem_columns <= 512
    assert r.flops == 2.0 * M * N * K * batch
    # never faster than the roofline it is derived from
    peak = 1663.5e12 / (6.0 if kwargs["dtype"] == "fp32" else 1.0)
    assert r.estimated_latency_ns * 1e-9 >= max(r.flops / peak, r.bytes / 6552e9)
    assert r.launch.grid == r.grid_dims


def test_plan_follows_the_dispatch_rules(lib):
    # fp32: the split-in-kernel variant only for small / batched shapes, otherwise pre-split planes (2 pre-pass kernels)
    small = planner.compile_matmul(512, 512, 512, dtype="fp32")
    big = planner.compile_matmul(4096, 4096, 4096, dtype="fp32")
    assert small.prepass_launches == 0 and small.workspace_bytes == 0
    assert big.prepass_launches == 2 and big.workspace_bytes >= 2 * 2 * 4096 * 4096 * 4
    # bf16: a leading dimension that is not a multiple of 8 elements forces a repack of that operand
    assert planner.compile_matmul(300, 304, 304, dtype="bf16").prepass_launches == 0
    assert planner.compile_matmul(300, 300, 300, dtype="bf16").prepass_launches == 2
    # cfg4 is HBM-bound, the big bf16 GEMMs are tensor-bound
    assert planner.compile_matmul(64, 64, 64, dtype="fp32", batch=2048).bound == "hbm"
    assert planner.compile_matmul(8192, 8192, 8192, dtype="bf16").bound == "tensor"
    # split-K over a cluster only when the tiles alone leave most SMs idle and K is long enough
    assert planner.compile_matmul(512, 512, 512, dtype="fp32").grid_dims[0] == 32 * 4
    assert planner.compile_matmul(512, 1024, 512, dtype="fp32").cluster_size == 2
    assert planner.compile_matmul(512, 512, 64, dtype="fp32").cluster_size == 1
    assert planner.compile_matmul(1024, 1024, 512, dtype="fp32").cluster_size == 1
    # mid-size bf16: pair tiles of 256x256 when the taller tile would only add padding or a wave
    assert planner.compile_matmul(256, 32768, 512, dtype="bf16").optimal_tile == (256, 256, 64)
    assert planner.compile_matmul(2048, 2048, 2048, dtype="bf16").optimal_tile == (256, 256, 64)   # 1 wave, not 2 of 128x128
    assert planner.compile_matmul(512, 512, 512, dtype="bf16").kernel_name == "gemm_tc_kernel"      # 32 small tiles > 4 pairs
    # stream-K is an option: off, a badly quantised shape takes whole tiles (here the 256x256 ones: 5 waves beat 3 of the
    # taller tile); on, every CTA pair of the device is busy on the 512x256 tiles and the plan says so
    off = planner.compile_matmul(4608, 4608, 4096, dtype="bf16", num_sms=148)
    assert off.optimal_tile == (256, 256, 64) and off.tiles == 18 * 18
    with _capi.option("stream_k", 1):
        on = planner.compile_matmul(4608, 4608, 4096, dtype="bf16", num_sms=148)
        tiny = planner.compile_matmul(1024, 512, 256, dtype="bf16", num_sms=148)  # 16 k-blocks in all: too short to share
    assert on.optimal_tile == (512, 256, 64) and on.tiles == 9 * 18 and on.grid_dims[0] == 148
    assert on.estimated_latency_ns < 1.2 * off.estimated_latency_ns
    assert tiny.grid_dims[0] < 148
    # fewer SMs -> smaller grid
    assert planner.compile_matmul(8192, 8192, 8192, dtype="bf16", num_sms=64).grid_dims[0] == 64


def test_invalid_requests_are_reported_in_the_result(lib):
    r = planner.compile_matmul(64, 64, 64, dtype="fp16")
    assert not r.valid and "in_dtype" in r.error
    r = planner.compile_matmul(0, 64, 64, dtype="bf16")
    assert not r.valid and "empty" in r.error
    r = planner.compile_matmul(64, 64, 64, dtype="bf16", activation="swish")
    assert not r.valid and "activation" in r.error


def test_cuda_compile_kernel_descriptions(lib):
    from symplex_b200 import engine
    k = engine.cuda_compile_kernel("matmul", {"M": 128, "N": 128, "K": 64, "tile_m": 32, "tile_n": 32, "tile_k": 8})
    assert k.kernel_name() == "gemm_f32_fused_kernel" and k.estimated_gflops() > 0 and k.ptx_size() == len(k.ptx_source())
    assert k.block_dims() == (448, 1, 1) and k.grid_dims()[0] == 2
    assert engine.cuda_compile_kernel("matmul", {"M": 64, "N": 128, "K": 64}).kernel_name() == "gemm_f32_small_kernel"
    e = engine.cuda_compile_kernel("elementwise", {"op": "add", "n": 1 << 24})
    assert e.kernel_name() == "fused_elementwise_ring_kernel" and e.block_dims() == (288, 1, 1)
    assert e.grid_dims()[0] == 148 * 2 and e.shared_mem_bytes() == 256 + 3 * 2 * 16384
    f = engine.cuda_compile_kernel("fma", {"n": 1 << 24})
    assert f.grid_dims()[0] == 148 * 3 and f.shared_mem_bytes() == 256 + 3 * 3 * 8192
    r = engine.cuda_compile_kernel("reduction", {"op": "max", "n": 1000})
    assert r.grid_dims()[0] == 1
    with pytest.raises(ValueError):
        engine.cuda_compile_kernel("elementwise", {"op": "pow", "n": 10})
    with pytest.raises(ValueError):
        engine.cuda_compile_kernel("reduction", {"op": "mul", "n": 10})
    with pytest.raises(ValueError):
        engine.cuda_compile_kernel("conv9d", {})
    assert "fused_elementwise_ring_kernel" in _symplex_core.cuda_compile_ptx("fma", {"n": 512})
