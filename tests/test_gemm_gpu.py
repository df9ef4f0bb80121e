"""Parity of the CUDA path against the CPU oracle, through the C ABI, on a B200.

Tolerances of the task statement: relative Frobenius error <= 1e-5 for the fp32 (3xTF32) path against the
reference's fp32 result, <= 1e-2 for bf16 inputs against the reference run on bf16-rounded inputs.
Large configurations are checked on a sample of rows (exact for a row-partitioned contraction) plus a
whole-output checksum identity.
"""
import ctypes

import numpy as np
import pytest
import torch

import symplex_b200 as sx
from oracle_loader import rel_frobenius
from symplex_b200 import _capi, _symplex_core as core, engine

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_BF16 = 1e-2
DEV = "cuda:0"


@pytest.fixture(scope="module", autouse=True)
def _require_gpu(lib):
    assert lib.symplex_cuda_available() == 1, "these tests need a B200 and the CUDA library (no fallback)"
    before = lib.symplex_b200_launch_count()
    yield
    assert lib.symplex_b200_launch_count() > before, "no kernel of the library was launched"
    assert lib.symplex_b200_sync_status(None) == 0


def _bf16_t(x_np):
    """numpy fp32 (already bf16-representable) -> torch bf16 on the GPU."""
    return torch.from_numpy(x_np).to(DEV).to(torch.bfloat16)


# ------------------------------------------------------------------ fp32 path, host-pointer drop-ins

def test_config1_fp32_512_cube(lib, oracle):
    """The fp32 512-cube: the shape the reference's own JIT-vs-NumPy bench runs."""
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    B = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    ref = oracle.jit_parallel_matmul(A, B)
    for fn in (core.jit_parallel_matmul, core.parallel_matmul, core.cuda_matmul):
        C = np.full((512, 512), np.nan, np.float32)
        assert fn(A.ctypes.data, B.ctypes.data, C.ctypes.data, 512, 512, 512) == 0
        assert rel_frobenius(C, ref) <= TOL_F32
    assert rel_frobenius(sx.matmul_jit(A, B), ref) <= TOL_F32
    assert rel_frobenius(sx.matmul_tiled(A, B), ref) <= TOL_F32


@pytest.mark.parametrize("shape", [
    (1, 1, 1), (2, 2, 2), (4, 4, 4), (3, 5, 7), (65, 33, 17), (128, 128, 128), (129, 257, 63), (1, 1000, 33),
    (1000, 1, 33), (300, 200, 1), (257, 129, 1025), (64, 64, 4096),
])
def test_fp32_shapes_against_oracle(lib, oracle, shape):
    M, N, K = shape
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    C = np.full((M, N), np.nan, np.float32)
    lib.symplex_matmul_f32(A.ctypes.data, B.ctypes.data, C.ctypes.data, M, N, K)
    assert not np.isnan(C).any()
    assert rel_frobenius(C, oracle.jit_parallel_matmul(A, B)) <= TOL_F32


def test_reference_known_answers_on_gpu(lib):
    A = np.array([[1, 2], [3, 4]], np.float32)
    B = np.array([[5, 6], [7, 8]], np.float32)
    np.testing.assert_array_equal(sx.matmul_jit(A, B), [[19, 22], [43, 50]])  # python/tests/test_jit.py:60-66
    Bm = np.arange(1, 17, dtype=np.float32).reshape(4, 4)
    np.testing.assert_allclose(sx.matmul_jit(np.eye(4, dtype=np.float32), Bm), Bm, atol=0.01)  # matmul_kernel.rs:1230
    a = (((np.arange(128 * 128) * 7 + 13) % 97) / 10.0).astype(np.float32).reshape(128, 128)   # matmul_bench.rs:39
    b = (((np.arange(128 * 128) * 11 + 17) % 89) / 10.0).astype(np.float32).reshape(128, 128)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    assert np.max(np.abs(sx.matmul_jit(a, b) - exact)) <= 0.01
    rng = np.random.default_rng(42)  # test_jit_native.py:60-78
    x, y = rng.standard_normal((32, 32)).astype(np.float32), rng.standard_normal((32, 32)).astype(np.float32)
    C = np.zeros((32, 32), np.float32)
    assert engine.MatmulKernel().execute_raw(x.ctypes.data, y.ctypes.data, C.ctypes.data, 32, 32, 32) == 0
    assert np.max(np.abs(C - x @ y)) < 1e-2


def test_golden_vectors_from_the_reference(lib, golden):
    for i in range(int(golden["mm_count"])):
        A, B = golden[f"mm{i}_A"], golden[f"mm{i}_B"]
        got = sx.matmul_jit(A, B)
        for key in ("py_matmul_jit", "c_matmul_f32", "c_matmul_tiled_f32"):
            assert rel_frobenius(got, golden[f"mm{i}_{key}"]) <= TOL_F32, (i, key)
    X, W, b = golden["fused_X"], golden["fused_W"], golden["fused_b"]
    assert rel_frobenius(sx.fused_matmul_bias_relu(X, W, b), golden["fused_relu"]) <= TOL_F32
    d = sx.make_desc(X.shape[0], W.shape[1], X.shape[1], activation="gelu")
    C = np.zeros((X.shape[0], W.shape[1]), np.float32)
    sx.gemm_host(d, X.ctypes.data, W.ctypes.data, C.ctypes.data, b.ctypes.data)
    assert rel_frobenius(C, golden["fused_gelu"]) <= TOL_F32


def test_fused_matmul_bias_relu_kernel_abi(lib, oracle):
    rng = np.random.default_rng(11)
    M, N, K = 200, 136, 300
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    ref = oracle.fused_matmul_bias_relu(A, B, bias)
    C = np.full((M, N), np.nan, np.float32)
    k = engine.FusedMatMulBiasReLUKernel()
    assert k.execute_raw(A.ctypes.data, B.ctypes.data, C.ctypes.data, bias.ctypes.data, M, N, K) == 0
    assert rel_frobenius(C, ref) <= TOL_F32
    assert np.all(C >= 0)
    C2 = np.zeros_like(C)
    assert lib.symplex_exec_fused_matmul_bias_relu(A.ctypes.data, B.ctypes.data, C2.ctypes.data, M, N, K,
                                                   bias.ctypes.data) == 0
    np.testing.assert_array_equal(C, C2)  # deterministic


def test_thin_sgemm_abi_and_fixed_dims_kernel(lib, oracle):
    rng = np.random.default_rng(12)
    A = rng.uniform(-1, 1, (96, 80)).astype(np.float32)
    B = rng.uniform(-1, 1, (80, 112)).astype(np.float32)
    ref = oracle.jit_parallel_matmul(A, B)
    for fn in (lib.blas_sgemm, lib.cache_tiled_sgemm_thin, lib.symplex_matmul_tiled_f32):
        C = np.full((96, 112), np.nan, np.float32)
        fn(A.ctypes.data, B.ctypes.data, C.ctypes.data, 96, 112, 80)
        assert rel_frobenius(C, ref) <= TOL_F32
    k = engine.AVX512MatmulKernel(96, 112, 80)
    C = np.full((96, 112), np.nan, np.float32)
    assert k.execute_raw(A.ctypes.data, B.ctypes.data, C.ctypes.data, 1, 1, 1) == 0  # runtime dims ignored
    assert rel_frobenius(C, ref) <= TOL_F32


def test_device_info_and_availability(lib):
    info = core.cuda_device_info()
    assert info["available"] is True and info["compute_capability_major"] == 10
    assert info["num_sms"] >= 100 and info["warp_size"] == 32 and info["total_memory_bytes"] > 100e9
    assert info["sm_arch"].startswith("sm_10") and "B200" in core.cuda_info()


# ------------------------------------------------------------------ device-pointer API

def _run(A_t, B_t, **kw):
    out = sx.gemm(A_t, B_t, **kw)
    sx.sync_status()
    return out


def test_config2_bf16_4096_colmajor_b(lib, oracle):
    """The bf16 4096-cube: row-major A, column-major B, fp32 output; oracle on 512 sampled rows."""
    rng = np.random.default_rng(2)
    n = 4096
    A = oracle.bf16_round(rng.standard_normal((n, n)).astype(np.float32))
    Bt = oracle.bf16_round(rng.standard_normal((n, n)).astype(np.float32))  # stored [N, K] = column-major B
    C = _run(_bf16_t(A), _bf16_t(Bt), b_layout=sx.COL_MAJOR, out_dtype=torch.float32).cpu().numpy()
    rows = np.sort(rng.choice(n, 512, replace=False))
    ref = oracle.matmul_rows(A, np.ascontiguousarray(Bt.T), rows)
    assert rel_frobenius(C[rows], ref) <= TOL_BF16
    assert rel_frobenius(C[rows], ref) <= 1e-5  # bf16 products are exact in fp32; only summation order differs
    _checksum_identity(C, A, Bt.T, 1e-5)


def test_config2_fp32_4096_via_3xtf32(lib, oracle):
    rng = np.random.default_rng(3)
    n = 4096
    A = rng.standard_normal((n, n)).astype(np.float32)
    Bt = rng.standard_normal((n, n)).astype(np.float32)
    C = _run(torch.from_numpy(A).to(DEV), torch.from_numpy(Bt).to(DEV), b_layout=sx.COL_MAJOR).cpu().numpy()
    rows = np.sort(rng.choice(n, 256, replace=False))
    ref = oracle.matmul_rows(A, np.ascontiguousarray(Bt.T), rows)
    assert rel_frobenius(C[rows], ref) <= TOL_F32
    _checksum_identity(C, A, Bt.T, 1e-5)


def _checksum_identity(C, A, B, tol):
    """Whole-output property: C.1 == A.(B.1) (evaluated in fp64)."""
    lhs = C.astype(np.float64).sum(axis=1)
    rhs = A.astype(np.float64) @ B.astype(np.float64).sum(axis=1)
    scale = np.linalg.norm(np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64).sum(axis=1))
    assert np.linalg.norm(lhs - rhs) / scale <= tol


def test_config3_fused_gelu_mlp_layer(lib, oracle):
    """The fused MLP layer Y = GELU(X.W + b), bf16 in/out, one kernel; oracle on 96 sampled rows."""
    rng = np.random.default_rng(4)
    M, K, N = 8192, 4096, 16384
    X = oracle.bf16_round(rng.normal(0, 0.02, (M, K)).astype(np.float32))
    W = oracle.bf16_round(rng.normal(0, 0.02, (K, N)).astype(np.float32))
    b = rng.normal(0, 0.02, N).astype(np.float32)
    before = sx.launch_count()
    Y = _run(_bf16_t(X), _bf16_t(W), bias=torch.from_numpy(b).to(DEV), activation="gelu")
    assert sx.launch_count() - before == 1, "the fused layer must be a single kernel"
    assert Y.dtype == torch.bfloat16
    rows = np.sort(rng.choice(M, 96, replace=False))
    ref = oracle.epilogue(oracle.matmul_rows(X, W, rows), bias=b, act=_capi.ACT_GELU)
    ref = oracle.bf16_round(ref)
    got = Y[torch.from_numpy(rows).to(DEV)].float().cpu().numpy()
    assert rel_frobenius(got, ref) <= TOL_BF16


def test_config4_batched_small_gemm(lib, oracle):
    """The batched small GEMM: 2048 independent fp32 64x64x64 problems, strided-batched."""
    rng = np.random.default_rng(5)
    nb = 2048
    A = rng.uniform(-1, 1, (nb, 64, 64)).astype(np.float32)
    B = rng.uniform(-1, 1, (nb, 64, 64)).astype(np.float32)
    C = _run(torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV)).cpu().numpy()
    ref = np.stack([oracle.jit_parallel_matmul(A[i], B[i], threads=1) for i in range(nb)])
    assert rel_frobenius(C, ref) <= TOL_F32
    worst = max(rel_frobenius(C[i], ref[i]) for i in range(0, nb, 37))
    assert worst <= TOL_F32


def test_config5_row_sharded_shape_on_one_gpu(lib, oracle):
    """The row-sharded product on one GPU: bf16 [65536, 8192] x [8192, 8192] -> bf16, no collective."""
    from symplex_b200.sharding import RowShardedGemm
    g = torch.Generator(device=DEV).manual_seed(6)
    M, N, K = 65536, 8192, 8192
    A = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    B = torch.randn(K, N, device=DEV, generator=g).to(torch.bfloat16)
    op = RowShardedGemm(M, N, K)
    assert op.world == 1 and op.chunks == 1
    C = op(A, B)
    sx.sync_status()
    rows = np.sort(np.random.default_rng(6).choice(M, 48, replace=False))
    rows_t = torch.from_numpy(rows).to(DEV)
    ref = oracle.bf16_round(oracle.matmul_rows(A[rows_t].float().cpu().numpy(), B.float().cpu().numpy(),
                                               np.arange(len(rows))))
    assert rel_frobenius(C[rows_t].float().cpu().numpy(), ref) <= TOL_BF16
    # whole-output checksum on the device in fp64: C.1 == A.(B.1), up to the bf16 rounding of C
    lhs = C.double().sum(dim=1)
    rhs = A.double() @ B.double().sum(dim=1)
    scale = (A.double().abs() @ B.double().abs().sum(dim=1)).norm()
    assert ((lhs - rhs).norm() / scale).item() <= 1e-3


@pytest.mark.parametrize("tile", [64, 128, 256])
@pytest.mark.parametrize("b_layout", [0, 1])
def test_bf16_tiles_and_layouts(lib, oracle, tile, b_layout):
    rng = np.random.default_rng(tile + b_layout)
    M, N, K = 384, 640, 520
    A = oracle.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    B = oracle.bf16_round(rng.standard_normal((K, N)).astype(np.float32))
    Bs = np.ascontiguousarray(B.T) if b_layout == sx.COL_MAJOR else B
    C = _run(_bf16_t(A), _bf16_t(Bs), b_layout=b_layout, out_dtype=torch.float32, tile_n=tile).cpu().numpy()
    assert rel_frobenius(C, oracle.jit_parallel_matmul(A, B)) <= 1e-5


@pytest.mark.parametrize("shape", [(1, 8, 8), (5, 3, 9), (130, 70, 17), (128, 256, 64), (100, 260, 33), (257, 8, 1000)])
@pytest.mark.parametrize("b_layout", [0, 1])
def test_bf16_ragged_and_unaligned(lib, oracle, shape, b_layout):
    """Shapes whose rows are not multiples of 16 bytes go through the padded-copy path."""
    M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    A = oracle.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    B = oracle.bf16_round(rng.standard_normal((K, N)).astype(np.float32))
    Bs = np.ascontiguousarray(B.T) if b_layout == sx.COL_MAJOR else B
    C = _run(_bf16_t(A), _bf16_t(Bs), b_layout=b_layout).float().cpu().numpy()
    ref = oracle.bf16_round(oracle.jit_parallel_matmul(A, B))
    assert rel_frobenius(C, ref) <= TOL_BF16


@pytest.mark.parametrize("offset", [1, 2, 3, 5, 7])
@pytest.mark.parametrize("shape", [(70, 40, 9), (130, 72, 33), (300, 264, 1001), (64, 128, 520)])
def test_bf16_operands_at_every_misalignment_equal_the_aligned_product(lib, shape, offset):
    """A and B start `offset` elements (2 bytes each) past a 16-byte boundary, rows of any pitch, a batch of two: the
    padded copies the library makes (aligned 16-byte loads shifted into place) must hold exactly the operands' values,
    so the product equals, bit for bit, the one from aligned, padded operands."""
    M, N, K = shape
    g = torch.Generator(device=DEV).manual_seed(M + K + offset)
    A = torch.randn(2, M, K, device=DEV, generator=g).to(torch.bfloat16)
    B = torch.randn(2, N, K, device=DEV, generator=g).to(torch.bfloat16)  # stored [N, K]
    bufA = torch.zeros(A.numel() + 16, device=DEV, dtype=torch.bfloat16)
    bufB = torch.full((B.numel() + 16,), float("nan"), device=DEV, dtype=torch.bfloat16)  # garbage around B
    Am = bufA[offset:offset + A.numel()].view(2, M, K)
    Bm = bufB[offset:offset + B.numel()].view(2, N, K)
    Am.copy_(A)
    Bm.copy_(B)
    assert Am.data_ptr() % 16 == (2 * offset) % 16 and Am.is_contiguous()
    got = _run(Am, Bm, b_layout=sx.COL_MAJOR, out_dtype=torch.float32)
    Kp = (K + 7) // 8 * 8  # the same values in rows padded to 16 bytes: no copy is made
    Ap = torch.zeros(2, M, Kp, device=DEV, dtype=torch.bfloat16)
    Bp = torch.zeros(2, N, Kp, device=DEV, dtype=torch.bfloat16)
    Ap[:, :, :K] = A
    Bp[:, :, :K] = B
    want = _run(Ap, Bp, b_layout=sx.COL_MAJOR, out_dtype=torch.float32)
    assert torch.equal(got, want)
    assert torch.isfinite(got).all()


@pytest.mark.parametrize("dtype,n", [(torch.bfloat16, 2048), (torch.bfloat16, 640), (torch.float32, 512),
                                     (torch.float32, 1536)])
def test_back_to_back_products_that_feed_each_other(lib, set_option, dtype, n):
    """Each product's output is the next one's A, launched back to back on one stream with no host synchronisation. The
    kernels start their set-up while their predecessor drains (programmatic dependent launch); they must not read an
    operand before the kernel that writes it has completed. The chain is compared, bit for bit, with the same chain
    run with that overlap switched off and a device synchronisation after every product."""
    g = torch.Generator(device=DEV).manual_seed(n)
    X = (torch.randn(n, n, device=DEV, generator=g) / 8).to(dtype)
    W = (torch.randn(n, n, device=DEV, generator=g) / (n ** 0.5)).to(dtype)  # keeps the chain's magnitude level

    bias0 = torch.zeros(n, device=DEV)

    def chain(sync):
        cur = X
        for i in range(8):
            # the previous product is this one's A and its residual (plain loads in the epilogue), and a row of it its bias
            bias = bias0 if i == 0 else cur[0].float().contiguous()
            cur = sx.gemm(cur, W, activation="tanh", residual=cur, beta=0.25, bias=bias)
            if sync:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        return cur

    set_option("pdl", 1)
    fast = [chain(False) for _ in range(3)]
    sx.sync_status()
    set_option("pdl", 0)
    want = chain(True)
    for got in fast:
        assert torch.equal(got, want)
    assert torch.isfinite(want.float()).all() and float(want.float().abs().max()) > 0


ACTS = [("none", 0), ("relu", 1), ("gelu", 2), ("sigmoid", 3), ("tanh", 4), ("silu", 5)]


@pytest.mark.parametrize("name,code", ACTS)
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_epilogue_chain(lib, oracle, name, code, dtype):
    """[MatMul, Mul, Add, act] with a residual: act(alpha * A.B + beta * R + bias)."""
    rng = np.random.default_rng(code)
    M, N, K = 200, 328, 136
    A = rng.normal(0, 0.5, (M, K)).astype(np.float32)
    B = rng.normal(0, 0.5, (K, N)).astype(np.float32)
    R = rng.normal(0, 1, (M, N)).astype(np.float32)
    bias = rng.normal(0, 1, N).astype(np.float32)
    alpha, beta = 0.75, -0.5
    if dtype == "bf16":
        A, B, R = oracle.bf16_round(A), oracle.bf16_round(B), oracle.bf16_round(R)
        mk = _bf16_t
    else:
        mk = lambda x: torch.from_numpy(x).to(DEV)
    out = _run(mk(A), mk(B), bias=torch.from_numpy(bias).to(DEV), residual=mk(R), activation=name,
               alpha=alpha, beta=beta).float().cpu().numpy()
    ref = oracle.epilogue(oracle.jit_parallel_matmul(A, B), alpha=alpha, beta=beta, residual=R, bias=bias, act=code)
    if dtype == "bf16":
        assert rel_frobenius(out, oracle.bf16_round(ref)) <= TOL_BF16
    else:
        assert rel_frobenius(out, ref) <= TOL_F32


def test_fp32_rowmajor_and_colmajor_b_agree(lib, oracle):
    rng = np.random.default_rng(21)
    M, N, K = 300, 200, 500
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    c_row = _run(torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV))
    c_col = _run(torch.from_numpy(A).to(DEV), torch.from_numpy(np.ascontiguousarray(B.T)).to(DEV),
                 b_layout=sx.COL_MAJOR)
    assert torch.equal(c_row, c_col)  # same planes, same kernel: bit-identical
    assert rel_frobenius(c_row.cpu().numpy(), oracle.jit_parallel_matmul(A, B)) <= TOL_F32


def test_fp32_accuracy_does_not_drift_with_k(lib, oracle):
    """Long reductions: the in-tensor-core accumulation is drained every 128 k, so error stays flat."""
    rng = np.random.default_rng(22)
    M, N, K = 128, 128, 16384
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    C = _run(torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV)).cpu().numpy()
    exact = A.astype(np.float64) @ B.astype(np.float64)
    assert rel_frobenius(C, exact) <= 2e-6
    assert rel_frobenius(C, oracle.jit_parallel_matmul(A, B)) <= TOL_F32


def test_linearity_property_full_size(lib):
    """(A1 + A2).B == A1.B + A2.B within fp32 rounding, at 4096^3 (no oracle needed)."""
    g = torch.Generator(device=DEV).manual_seed(23)
    n = 4096
    A1 = torch.randn(n, n, device=DEV, generator=g)
    A2 = torch.randn(n, n, device=DEV, generator=g)
    B = torch.randn(n, n, device=DEV, generator=g)
    lhs = _run(A1 + A2, B)
    rhs = _run(A1, B) + _run(A2, B)
    assert ((lhs - rhs).double().norm() / lhs.double().norm()).item() <= 5e-6


def test_caller_workspace_entry_point(lib, oracle):
    rng = np.random.default_rng(24)
    M, N, K = 256, 192, 320
    A = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(DEV)
    B = torch.from_numpy(rng.standard_normal((K, N)).astype(np.float32)).to(DEV)
    d = sx.make_desc(M, N, K)
    need = lib.symplex_b200_gemm_workspace_bytes(ctypes.byref(d))
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    C = torch.full((M, N), float("nan"), device=DEV)
    s = torch.cuda.current_stream().cuda_stream
    assert lib.symplex_b200_gemm_ws(ctypes.byref(d), A.data_ptr(), B.data_ptr(), C.data_ptr(), None, None,
                                    ws.data_ptr(), need, s) == 0
    assert lib.symplex_b200_gemm_ws(ctypes.byref(d), A.data_ptr(), B.data_ptr(), C.data_ptr(), None, None,
                                    ws.data_ptr(), need - 1, s) == _capi.ERR_INVALID
    sx.sync_status()
    assert torch.equal(C, sx.gemm(A, B))


def test_strided_host_output(lib, oracle):
    """ldc > N on the host path keeps the bytes between rows."""
    rng = np.random.default_rng(25)
    M, N, K, ldc = 40, 24, 16, 32
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    Cbuf = np.full((M, ldc), 9.0, np.float32)
    d = sx.make_desc(M, N, K, ldc=ldc)
    sx.gemm_host(d, A.ctypes.data, B.ctypes.data, Cbuf.ctypes.data)
    assert np.all(Cbuf[:, N:] == 9.0)
    assert rel_frobenius(Cbuf[:, :N], oracle.jit_parallel_matmul(A, B)) <= TOL_F32


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_host_path_row_chunked_pipeline(lib, oracle, dtype):
    """Large host-buffer problems are copied and computed in row chunks on three streams; the result must be the
    one the single-shot path gives (rows are independent)."""
    rng = np.random.default_rng(31)
    M, N, K = 8192 + 100, 384, 512
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    if dtype == "bf16":
        A_h = torch.from_numpy(A).to(torch.bfloat16)
        B_h = torch.from_numpy(B).to(torch.bfloat16)
        C_h = torch.empty(M, N, dtype=torch.bfloat16)
        d = sx.make_desc(M, N, K, sx.DT_BF16, sx.DT_BF16, activation="relu")
    else:
        A_h, B_h = torch.from_numpy(A), torch.from_numpy(B)
        C_h = torch.empty(M, N, dtype=torch.float32)
        d = sx.make_desc(M, N, K, activation="relu")
    results = []
    for name, value in (("pipeline_mb", 1), ("pipeline", 0)):
        with _capi.option(name, value):
            C_h.fill_(float("nan"))
            before = sx.launch_count()
            sx.gemm_host(d, A_h.data_ptr(), B_h.data_ptr(), C_h.data_ptr(), bias.ctypes.data)
            results.append((C_h.float().numpy().copy(), sx.launch_count() - before))
    (chunked, n_chunked), (single, n_single) = results
    assert n_chunked >= 4 * n_single - 4, "the chunked path should have launched one GEMM per row chunk"
    # Full chunks run the kernel the single-shot call runs: the same bits. The ragged last chunk (100 rows) is a
    # small problem of its own and, for fp32, goes to the split-K variant, whose summation order differs.
    np.testing.assert_array_equal(chunked[:8192], single[:8192])
    np.testing.assert_allclose(chunked[8192:], single[8192:], rtol=2e-5, atol=2e-5)
    rows = np.sort(rng.choice(M, 300, replace=False))
    Ar = oracle.bf16_round(A) if dtype == "bf16" else A
    Br = oracle.bf16_round(B) if dtype == "bf16" else B
    ref = oracle.epilogue(oracle.matmul_rows(Ar, Br, rows), bias=bias, act=_capi.ACT_RELU)
    tol = TOL_BF16 if dtype == "bf16" else TOL_F32
    assert rel_frobenius(chunked[rows], oracle.bf16_round(ref) if dtype == "bf16" else ref) <= tol


def test_headline_bf16_8192_cube_bias_gelu(lib, oracle):
    """The shape the 70 %-of-peak target is quoted on: 8192^3, bf16, bias + GELU fused, one kernel (exactly two waves
    of 512 x 256 pair tiles). Oracle on 64 sampled rows plus the whole-output checksum identity without the epilogue."""
    rng = np.random.default_rng(8192)
    n = 8192
    X = oracle.bf16_round(rng.normal(0, 0.02, (n, n)).astype(np.float32))
    W = oracle.bf16_round(rng.normal(0, 0.02, (n, n)).astype(np.float32))
    b = rng.normal(0, 0.02, n).astype(np.float32)
    tX, tW = _bf16_t(X), _bf16_t(W)
    before = sx.launch_count()
    Y = _run(tX, tW, bias=torch.from_numpy(b).to(DEV), activation="gelu")
    assert sx.launch_count() - before == 1
    rows = np.sort(rng.choice(n, 64, replace=False))
    ref = oracle.bf16_round(oracle.epilogue(oracle.matmul_rows(X, W, rows), bias=b, act=_capi.ACT_GELU))
    got = Y[torch.from_numpy(rows).to(DEV)].float().cpu().numpy()
    assert rel_frobenius(got, ref) <= TOL_BF16
    plain = _run(tX, tW, out_dtype=torch.float32).cpu().numpy()
    _checksum_identity(plain, X, W, 1e-5)


@pytest.mark.parametrize("chain,alpha", [
    (["matmul", "mul", "add", "gelu"], 0.5), (["matmul", "add", "relu"], 1.0), (["matmul", "silu"], 1.0),
    (["matmul", "add"], 1.0), (["matmul", "mul", "add", "tanh", "softmax"], 2.0),
])
def test_fusion_chain_to_descriptor_to_kernel(lib, oracle, chain, alpha):
    """An op list goes through the library's fusion discovery (symplex_b200_discover_fusions), the matched chain is
    compiled into the epilogue fields of a descriptor (symplex_b200_compile_epilogue), and that descriptor runs as
    ONE kernel whose result is the oracle's matmul followed by the same ops."""
    import json
    M, N, K = 384, 320, 200
    rng = np.random.default_rng(len(chain))
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    ops = [(name, [M, N], "fp32") for name in chain]
    arr, _keep = _capi.pack_fusion_ops(ops)
    buf = ctypes.create_string_buffer(4096)
    assert lib.symplex_b200_discover_fusions(arr, len(ops), buf, 4096) > 0
    found = json.loads(buf.value.decode())["boundaries"]
    d = sx.make_desc(M, N, K)
    consumed, has_bias, has_scale = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    assert lib.symplex_b200_compile_epilogue(arr, len(ops), 0, ctypes.byref(d), ctypes.byref(consumed),
                                             ctypes.byref(has_bias), ctypes.byref(has_scale)) == 0
    fusable = [c for c in chain if c != "softmax"]
    assert consumed.value == len(fusable)
    assert [b["op_indices"] for b in found] == [list(range(len(fusable)))] and found[0]["pattern"] == "MatMulBiasReLU"
    assert bool(has_bias.value) == ("add" in chain) and bool(has_scale.value) == ("mul" in chain)
    if has_scale.value:
        d.alpha = alpha
    tA, tB = torch.from_numpy(A).to(DEV), torch.from_numpy(B).to(DEV)
    tb = torch.from_numpy(bias).to(DEV)
    C = torch.full((M, N), float("nan"), device=DEV)
    before = sx.launch_count()
    rc = lib.symplex_b200_gemm(ctypes.byref(d), tA.data_ptr(), tB.data_ptr(), C.data_ptr(),
                               tb.data_ptr() if has_bias.value else None, None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _capi.last_error()
    sx.sync_status()
    assert sx.launch_count() - before == 1
    ref = oracle.epilogue(oracle.jit_parallel_matmul(A, B), alpha=alpha if has_scale.value else 1.0,
                          bias=bias if has_bias.value else None, act=d.activation)
    assert rel_frobenius(C.cpu().numpy(), ref) <= TOL_F32


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(1024, 768, 320), (600, 520, 136), (4096, 2048, 512)])
def test_peer_outputs_receive_every_tile(lib, shape, out_dtype):
    """The multi-destination epilogue on one GPU: two extra buffers stand in for other GPUs' C."""
    M, N, K = shape
    g = torch.Generator(device=DEV).manual_seed(41)
    A = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    B = torch.randn(K, N, device=DEV, generator=g).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV, generator=g)
    want = _run(A, B, bias=bias, activation="silu", out_dtype=out_dtype)
    peers = [torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype) for _ in range(2)]
    got = _run(A, B, bias=bias, activation="silu", out_dtype=out_dtype, peer_outputs=[p.data_ptr() for p in peers])
    assert torch.equal(got, want)
    for p in peers:
        assert torch.equal(p, want)


def test_tma_store_and_direct_store_epilogues_agree(lib):
    g = torch.Generator(device=DEV).manual_seed(42)
    A = torch.randn(2048, 512, device=DEV, generator=g).to(torch.bfloat16)
    B = torch.randn(512, 1000, device=DEV, generator=g).to(torch.bfloat16)  # ragged N: TMA clips the last block
    staged = _run(A, B, activation="gelu")
    with _capi.option("tma_store", 0):
        direct = _run(A, B, activation="gelu")
    assert torch.equal(staged, direct)


@pytest.mark.parametrize("ety,rhs_layout", [(9, 0), (9, 1), (11, 0), (11, 1)])
def test_tensor_matmul_wire_record(lib, oracle, ety, rhs_layout):
    """A serialized Instr::TensorMatMul (34-byte 0xA2 record) executed against a slot array of host pointers;
    the rhs layout byte is honoured."""
    import struct
    rng = np.random.default_rng(51 + ety + rhs_layout)
    M, N, K = 96, 136, 200
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    if ety == 11:
        A, B = oracle.bf16_round(A), oracle.bf16_round(B)
        to_dev = lambda x: oracle.f32_to_bf16_bits(x)
        C = np.zeros((M, N), np.uint16)
    else:
        to_dev = lambda x: x
        C = np.full((M, N), np.nan, np.float32)
    a_buf = np.ascontiguousarray(to_dev(A))
    b_buf = np.ascontiguousarray(to_dev(B.T if rhs_layout == 1 else B))
    rec = struct.pack("<BHHHQQQBBB", 0xA2, 3, 1, 2, M, N, K, ety, 0, rhs_layout)
    slots = (ctypes.c_void_p * 4)(None, a_buf.ctypes.data, b_buf.ctypes.data, C.ctypes.data)
    assert lib.symplex_b200_exec_tensor_matmul(rec, len(rec), slots, 4) == 0, _capi.last_error()
    ref = oracle.jit_parallel_matmul(A, B)
    if ety == 11:
        assert rel_frobenius(oracle.bf16_bits_to_f32(C), oracle.bf16_round(ref)) <= TOL_BF16
    else:
        assert rel_frobenius(C, ref) <= TOL_F32


@pytest.mark.parametrize("M,N,K,dtype,batch", [
    (512, 512, 512, "fp32", 1), (64, 64, 64, "fp32", 64), (2048, 1536, 1024, "fp32", 1),
    (300, 300, 300, "bf16", 1), (2048, 2048, 2048, "bf16", 1), (4096, 4096, 1024, "bf16", 1),
    (8192, 4096, 512, "bf16", 1),
])
def test_plan_describes_what_is_launched(lib, M, N, K, dtype, batch):
    """symplex_b200_gemm_plan and the launch path share one decision function: the number of kernels a call
    launches must be the plan's pre-pass count + 1, and the plan's latency estimate must be within a factor of
    three of the measured time (it is a roofline model, not a simulator)."""
    from symplex_b200 import planner
    plan = planner.compile_matmul(M, N, K, dtype=dtype, batch=batch)
    assert plan.valid
    tdt = torch.float32 if dtype == "fp32" else torch.bfloat16
    shape_a = (batch, M, K) if batch > 1 else (M, K)
    shape_b = (batch, K, N) if batch > 1 else (K, N)
    A = torch.randn(shape_a, device="cuda").to(tdt)
    B = torch.randn(shape_b, device="cuda").to(tdt)
    out = sx.gemm(A, B)
    before = sx.launch_count()
    sx.gemm(A, B, out=out)
    assert sx.launch_count() - before == plan.prepass_launches + 1
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(10):
        sx.gemm(A, B, out=out)
    e1.record()
    torch.cuda.synchronize()
    sx.sync_status()
    measured_ns = e0.elapsed_time(e1) / 10 * 1e6
    assert plan.estimated_latency_ns / 3 <= measured_ns <= plan.estimated_latency_ns * 3, (measured_ns, plan)


@pytest.mark.parametrize("split", [1, 2, 4])
@pytest.mark.parametrize("M,N,K,batch", [
    (512, 512, 512, 1),      # the fp32 512-cube: 32 tiles, 16 k-blocks
    (128, 64, 8192, 1),      # one tile, long K
    (200, 100, 300, 1),      # ragged edges; 10 k-blocks split 3,3,2,2
    (96, 64, 1056, 100),     # 100 tiles on 37 clusters: each cluster loops over several tiles
])
def test_fp32_split_k_over_a_cluster(lib, oracle, set_option, split, M, N, K, batch):
    """The cluster split-K variants of the fused fp32 kernel (partials exchanged over distributed shared memory)
    must meet the same 1e-5 bound as the unsplit kernel, with and without a fused epilogue, for both B layouts."""
    set_option("f32_split_k", split)
    rng = np.random.default_rng(7)
    shape_a = (batch, M, K) if batch > 1 else (M, K)
    shape_b = (batch, K, N) if batch > 1 else (K, N)
    A = rng.uniform(-1, 1, shape_a).astype(np.float32)
    B = rng.uniform(-1, 1, shape_b).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    tA, tB, tb = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), torch.from_numpy(bias).cuda()
    got = sx.gemm(tA, tB, bias=tb, activation="relu").cpu().numpy()
    tBt = tB.transpose(-1, -2).contiguous()
    got_col = sx.gemm(tA, tBt, b_layout=sx.COL_MAJOR).cpu().numpy()
    sx.sync_status()
    if batch > 1:
        sel = [0, 1, batch // 2, batch - 1]
        ref = np.stack([oracle.jit_parallel_matmul(A[z], B[z]) for z in sel])
        got, got_col = got[sel], got_col[sel]
    else:
        ref = oracle.jit_parallel_matmul(A, B)
    assert rel_frobenius(got_col, ref) <= 1e-5
    assert rel_frobenius(got, np.maximum(ref + bias, 0)) <= 1e-5


def test_fp32_split_k_is_reproducible(lib, set_option):
    set_option("f32_split_k", 4)
    A = torch.randn(256, 2048, device="cuda")
    B = torch.randn(2048, 128, device="cuda")
    first = sx.gemm(A, B)
    for _ in range(5):
        assert torch.equal(sx.gemm(A, B), first)
    sx.sync_status()


@pytest.mark.parametrize("M,N,K,batch", [(64, 64, 64, 8), (1, 64, 32, 1), (17, 100, 72, 3), (64, 320, 1000, 2), (40, 64, 4096, 1),
                                         (48, 2048, 256, 1)])
def test_fp32_64_row_mma_shape(lib, oracle, set_option, M, N, K, batch):
    """Problems with at most 64 rows run the M = 64 shape of the tensor-core instruction (accumulator rows in
    lanes 0-15 of each tensor-memory quarter). It must give the bits the 128-row shape gives (the zero rows that
    shape pads with contribute nothing) and meet the 1e-5 bound."""
    rng = np.random.default_rng(11)
    shape_a = (batch, M, K) if batch > 1 else (M, K)
    shape_b = (batch, K, N) if batch > 1 else (K, N)
    A = rng.uniform(-1, 1, shape_a).astype(np.float32)
    B = rng.uniform(-1, 1, shape_b).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    tA, tB, tb = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), torch.from_numpy(bias).cuda()
    out = {}
    set_option("f32_split_k", 1)
    for rows in ("64", "128"):
        set_option("f32_tile_rows", int(rows))
        out[rows] = (sx.gemm(tA, tB, bias=tb, activation="tanh").cpu().numpy(),
                     sx.gemm(tA, tB.transpose(-1, -2).contiguous(), b_layout=sx.COL_MAJOR,
                             out_dtype=torch.bfloat16).float().cpu().numpy())
    sx.sync_status()
    assert np.array_equal(out["64"][0], out["128"][0]) and np.array_equal(out["64"][1], out["128"][1])
    A2, B2 = (A[0], B[0]) if batch > 1 else (A, B)
    ref = oracle.jit_parallel_matmul(A2, B2)
    got, got_bf = (out["64"][0][0], out["64"][1][0]) if batch > 1 else out["64"]
    assert rel_frobenius(got, np.tanh(ref + bias)) <= 1e-5
    assert rel_frobenius(got_bf, oracle.bf16_round(ref)) <= 1e-2


@pytest.mark.parametrize("seed", range(24))
def test_random_configurations_against_oracle(lib, oracle, seed):
    """Seeded random sweep over everything the descriptor can say: dtype, ragged M / N / K, batch, B layout, bias,
    scale, activation, output dtype. Which kernel serves a case is the dispatcher's business; the oracle bound is
    the same for all of them."""
    rng = np.random.default_rng(1000 + seed)
    f32 = bool(rng.integers(0, 2))
    M, N, K = (int(rng.integers(1, 400)), int(rng.integers(1, 400)), int(rng.integers(1, 700)))
    if seed % 6 == 0:
        M = int(rng.integers(1, 65))  # the small-row kernel
    batch = int(rng.choice([1, 1, 2, 3, 5]))
    col_major = bool(rng.integers(0, 2))
    act = [None, "relu", "gelu", "sigmoid", "tanh", "silu"][int(rng.integers(0, 6))]
    use_bias = bool(rng.integers(0, 2))
    alpha = float(rng.choice([1.0, 0.5, -2.0]))
    out_bf16 = (not f32) and bool(rng.integers(0, 2))
    A = rng.uniform(-1, 1, (batch, M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (batch, K, N)).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32) if use_bias else None
    if not f32:
        A, B = oracle.bf16_round(A), oracle.bf16_round(B)
    tdt = torch.float32 if f32 else torch.bfloat16
    tA = torch.from_numpy(A).to(DEV).to(tdt)
    tB = torch.from_numpy(B).to(DEV).to(tdt)
    if col_major:
        tB = tB.transpose(-1, -2).contiguous()
    if batch == 1:
        tA, tB = tA[0], tB[0]
    got = sx.gemm(tA, tB, bias=torch.from_numpy(bias).to(DEV) if use_bias else None, activation=act, alpha=alpha,
                  b_layout=sx.COL_MAJOR if col_major else sx.ROW_MAJOR,
                  out_dtype=torch.bfloat16 if out_bf16 else torch.float32)
    sx.sync_status()
    got = got.float().cpu().numpy().reshape(batch, M, N)
    for z in range(batch):
        ref = oracle.epilogue(oracle.jit_parallel_matmul(A[z], B[z]), alpha=alpha, bias=bias,
                              act=_capi.ACTIVATIONS[act])
        if out_bf16:
            ref = oracle.bf16_round(ref)
        tol = TOL_F32 if f32 else TOL_BF16
        err = rel_frobenius(got[z], ref)
        assert err <= tol, dict(seed=seed, f32=f32, shape=(batch, M, N, K), col_major=col_major, act=act, bias=use_bias,
                                alpha=alpha, out_bf16=out_bf16, err=err)


def test_small_row_kernel_unaligned_output_and_odd_batch(lib, oracle):
    """N = 101 makes the rows of C 404 bytes long, so the TMA-store epilogue is not available and the kernel stores
    directly; an odd batch leaves the last pair half empty; M = 30 leaves two epilogue warps without rows."""
    rng = np.random.default_rng(5)
    batch, M, N, K = 3, 30, 101, 72
    A = rng.uniform(-1, 1, (batch, M, K)).astype(np.float32)
    Bt = rng.uniform(-1, 1, (batch, N, K)).astype(np.float32)  # column-major B: [N, K]
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    from symplex_b200 import planner
    assert planner.compile_matmul(M, N, K, dtype="fp32", batch=batch, b_layout=sx.COL_MAJOR).kernel_name == \
        "gemm_f32_small_kernel"
    got = sx.gemm(torch.from_numpy(A).cuda(), torch.from_numpy(Bt).cuda(), bias=torch.from_numpy(bias).cuda(),
                  activation="relu", b_layout=sx.COL_MAJOR).cpu().numpy()
    sx.sync_status()
    for z in range(batch):
        ref = np.maximum(oracle.jit_parallel_matmul(A[z], np.ascontiguousarray(Bt[z].T)) + bias, 0)
        assert rel_frobenius(got[z], ref) <= TOL_F32


def test_execute_with_kernel_args(lib, oracle):
    """The ORCJIT::execute-shaped entry point (jit::KernelArgs bundle, host pointers, fp32), plain and fused."""
    from test_capi_cpu import _kernel_args
    rng = np.random.default_rng(3)
    batch, M, N, K = 3, 70, 96, 130
    A = rng.uniform(-1, 1, (batch, M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (batch, K, N)).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    C = np.full((batch, M, N), np.nan, np.float32)
    assert lib.symplex_b200_execute(b"symplex_matmul_70x96x130", ctypes.byref(_kernel_args([A, B], C, M, N, K, batch))) == 0
    for z in range(batch):
        assert rel_frobenius(C[z], oracle.jit_parallel_matmul(A[z], B[z])) <= TOL_F32
    C1 = np.full((M, N), np.nan, np.float32)
    ka = _kernel_args([A[0], B[0], bias], C1, M, N, K, 1, sizes=False)
    assert lib.symplex_b200_execute(b"fused_matmul_bias_relu", ctypes.byref(ka)) == 0
    assert rel_frobenius(C1, oracle.fused_matmul_bias_relu(A[0], B[0], bias)) <= TOL_F32
