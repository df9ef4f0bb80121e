"""The f64 twins of the thin GEMM ABI (blas_dgemm / cache_tiled_dgemm_thin, rust-engine/src/phase3_jit.rs:449-461,
676-685) on the GPU: bit for bit the summation order of the reference's cache_tiled_dgemm, restated by the oracle."""
import ctypes
import struct

import numpy as np
import pytest
import torch

from oracle_loader import rel_frobenius
from symplex_b200 import _capi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(1, 1, 1), (2, 2, 2), (64, 64, 64), (65, 33, 17), (100, 70, 129), (37, 300, 500),
                                   (256, 192, 1000), (3, 5, 4097)])
def test_dgemm_host_entry_points_match_the_reference_order_exactly(lib, oracle, shape):
    M, N, K = shape
    rng = np.random.default_rng(M + 31 * N + 977 * K)
    A, B = rng.standard_normal((M, K)), rng.standard_normal((K, N))
    want = oracle.cache_tiled_dgemm(A, B)
    for fn in (lib.blas_dgemm, lib.cache_tiled_dgemm_thin):
        C = np.full((M, N), np.nan)
        fn(A.ctypes.data, B.ctypes.data, C.ctypes.data, M, N, K)
        np.testing.assert_array_equal(C, want)
    assert rel_frobenius(want, A @ B) <= 1e-14


def test_dgemm_device_entry_point_and_strides(lib, oracle):
    M, N, K = 130, 90, 260
    rng = np.random.default_rng(3)
    Abig, Bbig = rng.standard_normal((M, K + 7)), rng.standard_normal((K, N + 3))
    tA, tB = torch.from_numpy(Abig).cuda(), torch.from_numpy(Bbig).cuda()
    tC = torch.full((M, N + 5), float("nan"), device="cuda", dtype=torch.float64)
    s = torch.cuda.current_stream().cuda_stream
    rc = lib.symplex_b200_dgemm(tA.data_ptr(), tB.data_ptr(), tC.data_ptr(), M, N, K, K + 7, N + 3, N + 5, s)
    assert rc == 0, _capi.last_error()
    torch.cuda.synchronize()
    got = tC.cpu().numpy()
    np.testing.assert_array_equal(got[:, :N], oracle.cache_tiled_dgemm(Abig[:, :K], Bbig[:, :N]))
    assert np.isnan(got[:, N:]).all(), "columns beyond N must not be written"
    assert lib.symplex_b200_dgemm(tA.data_ptr(), tB.data_ptr(), tC.data_ptr(), M, N, K, K - 1, 0, 0, s) == _capi.ERR_INVALID


def test_dgemm_zero_k_and_zero_rows(lib):
    C = np.full((4, 3), np.nan)
    A, B = np.zeros((4, 0)), np.zeros((0, 3))
    lib.blas_dgemm(A.ctypes.data, B.ctypes.data, C.ctypes.data, 4, 3, 0)
    np.testing.assert_array_equal(C, np.zeros((4, 3)))  # the reference's loop nest zeroes C first
    C2 = np.full((2, 2), 7.0)
    lib.blas_dgemm(A.ctypes.data, B.ctypes.data, C2.ctypes.data, 0, 2, 5)
    np.testing.assert_array_equal(C2, np.full((2, 2), 7.0))


def test_tensor_matmul_record_with_f64_elements(lib, oracle):
    """The wire record of Instr::TensorMatMul with element type F64 (10): what the reference lowers to blas_dgemm."""
    M, N, K = 48, 40, 200
    rng = np.random.default_rng(4)
    A, B = rng.standard_normal((M, K)), rng.standard_normal((K, N))
    C = np.full((M, N), np.nan)
    rec = struct.pack("<BHHHQQQBBB", 0xA2, 2, 0, 1, M, N, K, _capi.DT_F64, 0, 0)
    slots = (ctypes.c_void_p * 3)(A.ctypes.data, B.ctypes.data, C.ctypes.data)
    assert lib.symplex_b200_exec_tensor_matmul(rec, len(rec), slots, 3) == 0, _capi.last_error()
    np.testing.assert_array_equal(C, oracle.cache_tiled_dgemm(A, B))
    rec = struct.pack("<BHHHQQQBBB", 0xA2, 2, 0, 1, M, N, K, _capi.DT_F64, 0, 1)
    assert lib.symplex_b200_exec_tensor_matmul(rec, len(rec), slots, 3) == _capi.ERR_INVALID  # col-major rhs
