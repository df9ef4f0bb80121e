"""C-ABI checks that need no GPU: the library loads, exports every symbol the header declares,
validates descriptors, and fails loudly (no CPU fallback) when asked to compute without a B200."""
import ctypes
import os
import re

import numpy as np
import pytest

from symplex_b200 import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "symplex_b200.h")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = "\n".join(line for line in text.splitlines() if not line.lstrip().startswith("#"))
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}]*\)\s*;", text)
    return sorted(set(n for n in names if n.startswith(("symplex_", "blas_", "cache_tiled_", "poly_"))))


def test_header_declares_functions():
    names = _declared_functions()
    assert "symplex_b200_gemm" in names and "symplex_matmul_f32" in names and "blas_sgemm" in names
    assert len(names) >= 19


def test_library_exports_every_declared_symbol(lib):
    for name in _declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/symplex_b200.h but not exported"


def test_binding_table_matches_header():
    assert sorted(_capi.SIGNATURES) == _declared_functions()


def test_desc_struct_layout(lib):
    # 3*8 + 4*4 + 6*8 + 2*4 + 2*4 = 104 bytes, no padding surprises
    assert ctypes.sizeof(_capi.GemmDesc) == 104
    d = _capi.GemmDesc()
    lib.symplex_b200_gemm_desc_init(ctypes.byref(d), 5, 6, 7, _capi.DT_F32, _capi.DT_BF16)
    assert (d.M, d.N, d.K, d.batch, d.in_dtype, d.out_dtype) == (5, 6, 7, 1, 9, 11)
    assert (d.alpha, d.beta, d.activation, d.b_layout, d.tile_n) == (1.0, 0.0, 0, 0, 0)


def test_workspace_sizes(lib):
    d = _capi.GemmDesc()
    lib.symplex_b200_gemm_desc_init(ctypes.byref(d), 512, 512, 512, _capi.DT_F32, _capi.DT_F32)
    # fp32: {hi, lo} planes of A [512x512] and of B [512x512]
    assert lib.symplex_b200_gemm_workspace_bytes(ctypes.byref(d)) == 2 * 2 * 512 * 512 * 4
    d.batch = 3
    assert lib.symplex_b200_gemm_workspace_bytes(ctypes.byref(d)) == 3 * 2 * 2 * 512 * 512 * 4
    lib.symplex_b200_gemm_desc_init(ctypes.byref(d), 65, 33, 17, _capi.DT_F32, _capi.DT_F32)
    a = 2 * 65 * 20 * 4
    b = 2 * 33 * 20 * 4
    assert lib.symplex_b200_gemm_workspace_bytes(ctypes.byref(d)) == (a + 255) // 256 * 256 + (b + 255) // 256 * 256
    lib.symplex_b200_gemm_desc_init(ctypes.byref(d), 128, 256, 64, _capi.DT_BF16, _capi.DT_BF16)
    assert lib.symplex_b200_gemm_workspace_bytes(ctypes.byref(d)) > 0  # worst case: unaligned pointers


@pytest.mark.parametrize("field,value", [
    ("in_dtype", 3), ("out_dtype", 10), ("b_layout", 2), ("activation", 6), ("activation", -1), ("tile_n", 32),
    ("M", -1), ("lda", 3),
])
def test_descriptor_validation(lib, field, value):
    d = _capi.GemmDesc()
    lib.symplex_b200_gemm_desc_init(ctypes.byref(d), 64, 64, 64, _capi.DT_F32, _capi.DT_F32)
    setattr(d, field, value)
    buf = (ctypes.c_float * 4096)()
    rc = lib.symplex_b200_gemm(ctypes.byref(d), buf, buf, buf, None, None, None)
    assert rc == _capi.ERR_INVALID
    assert lib.symplex_b200_gemm_workspace_bytes(ctypes.byref(d)) == 0
    assert len(_capi.last_error()) > 0


def test_null_descriptor(lib):
    assert lib.symplex_b200_gemm(None, None, None, None, None, None, None) == _capi.ERR_INVALID


def test_zero_dimension_is_a_noop(lib):
    # python/src/lib.rs:1030,1044,1839: zero dimension returns 0 before touching anything
    C = np.full((4, 4), 7.0, np.float32)
    for fn in (lib.symplex_parallel_matmul, lib.symplex_jit_parallel_matmul, lib.symplex_cuda_matmul,
               lib.symplex_exec_matmul):
        assert fn(None, None, C.ctypes.data, 4, 4, 0) == 0
        assert fn(None, None, C.ctypes.data, 0, 4, 4) == 0
    assert np.all(C == 7.0)
    # kernels/matmul.c zeroes C before accumulating over an empty k range
    A = np.zeros((4, 0), np.float32)
    lib.symplex_matmul_f32(A.ctypes.data, A.ctypes.data, C.ctypes.data, 4, 4, 0)
    assert np.all(C == 0.0)


def test_python_mirror_argument_errors():
    import symplex_b200 as sx
    with pytest.raises(ValueError, match="requires 2D arrays"):
        sx.matmul_jit(np.zeros(3, np.float32), np.zeros((3, 3), np.float32))
    with pytest.raises(ValueError, match="Shape mismatch"):
        sx.matmul_jit(np.zeros((2, 3), np.float32), np.zeros((4, 2), np.float32))
    with pytest.raises(ValueError):
        sx.make_desc(2, 2, 2, activation="swish")
    from symplex_b200 import engine
    with pytest.raises(ValueError):
        engine.AVX512MatmulKernel(0, 4, 4)
    assert engine.AVX512MatmulKernel(2, 3, 4).dims() == (2, 3, 4)


def _has_gpu():
    try:
        return bool(_capi.load().symplex_cuda_available())
    except Exception:
        return False


@pytest.mark.skipif(_has_gpu(), reason="checks the no-GPU failure path")
def test_no_gpu_fails_loudly_never_computes(lib):
    """Without a B200 nothing is computed on the host: error codes out, C untouched."""
    import symplex_b200 as sx
    from symplex_b200 import _symplex_core as core
    A = np.ones((8, 8), np.float32)
    C = np.full((8, 8), -3.0, np.float32)
    assert core.cuda_available() is False
    assert core.cuda_matmul(A.ctypes.data, A.ctypes.data, C.ctypes.data, 8, 8, 8) == -1
    assert core.jit_parallel_matmul(A.ctypes.data, A.ctypes.data, C.ctypes.data, 8, 8, 8) < 0
    assert np.all(C == -3.0)
    # the void drop-ins cannot return a code: they poison C and leave the reason
    lib.symplex_matmul_f32(A.ctypes.data, A.ctypes.data, C.ctypes.data, 8, 8, 8)
    assert np.isnan(C).all() and _capi.last_error() != "no error"
    D = np.full((8, 8), -3.0)
    Ad = np.ones((8, 8))
    lib.blas_dgemm(Ad.ctypes.data, Ad.ctypes.data, D.ctypes.data, 8, 8, 8)
    assert np.isnan(D).all()
    info = core.cuda_device_info()
    assert info["available"] is False and "error" in info
    with pytest.raises(sx.SymplexB200Error):
        sx.matmul_jit(A, A)
    with pytest.raises(sx.SymplexB200Error):
        sx.matmul_tiled(A, A)
    with pytest.raises(sx.SymplexB200Error):
        sx.fused_matmul_bias_relu(A, A, np.zeros(8, np.float32))


def test_missing_library_raises(monkeypatch, tmp_path):
    monkeypatch.setattr(_capi, "_lib", None)
    monkeypatch.setattr(_capi, "LIB_PATH", str(tmp_path / "libsymplex_b200.so"))
    with pytest.raises(ImportError, match="no CPU fallback"):
        _capi.load()


def test_struct_sizes_match_the_compiled_library(lib):
    sizes = (ctypes.c_int32 * 5)()
    lib.symplex_b200_abi_sizes(ctypes.byref(sizes))
    assert list(sizes) == [ctypes.sizeof(t) for t in (_capi.GemmDesc, _capi.DeviceInfo, _capi.FusedOp, _capi.Target,
                                                      _capi.GemmPlan)]
    assert sizes[0] == 104 and sizes[2] == 8


def _kernel_args(arrays, out, M, N, K, batch=1, sizes=True):
    ka = _capi.KernelArgs()
    ptrs = (ctypes.c_void_p * max(len(arrays), 1))(*[a.ctypes.data for a in arrays])
    szs = (ctypes.c_int64 * max(len(arrays), 1))(*[a.nbytes for a in arrays])
    ka.data, ka.data_size = out.ctypes.data, out.nbytes
    ka.input_ptrs, ka.num_inputs = ptrs, len(arrays)
    ka.input_sizes = szs if sizes else None
    ka.M, ka.N, ka.K, ka.batch = M, N, K, batch
    ka._keep = (ptrs, szs)
    return ka


def test_execute_kernel_args_validation(lib):
    """ORCJIT::execute-shaped entry point: struct layout of jit::KernelArgs and argument checks (no GPU needed)."""
    assert ctypes.sizeof(_capi.KernelArgs) == 9 * 8
    A, B, C = np.zeros((4, 6), np.float32), np.zeros((6, 5), np.float32), np.zeros((4, 5), np.float32)
    ok = _kernel_args([A, B], C, 4, 5, 6)
    assert lib.symplex_b200_execute(b"conv2d_3x3", ctypes.byref(ok)) == _capi.ERR_INVALID
    assert "not on this path" in _capi.last_error()
    assert lib.symplex_b200_execute(b"symplex_fused_matmul_bias_relu_4x5x6", ctypes.byref(ok)) == _capi.ERR_INVALID
    assert "takes 3 inputs" in _capi.last_error()
    small_out = _kernel_args([A, B], np.zeros(3, np.float32), 4, 5, 6)
    assert lib.symplex_b200_execute(b"matmul", ctypes.byref(small_out)) == _capi.ERR_INVALID
    assert "output holds 12 bytes" in _capi.last_error()
    small_in = _kernel_args([A[:2], B], C, 4, 5, 6)
    assert lib.symplex_b200_execute(b"matmul", ctypes.byref(small_in)) == _capi.ERR_INVALID
    assert "input 0 holds" in _capi.last_error()
    assert lib.symplex_b200_execute(b"matmul", ctypes.byref(_kernel_args([A, B], C, 0, 5, 6))) == 0   # nothing to do
    assert lib.symplex_b200_execute(b"matmul", None) == _capi.ERR_INVALID
    if not lib.symplex_cuda_available():
        assert lib.symplex_b200_execute(b"symplex_matmul_4x5x6", ctypes.byref(ok)) == _capi.ERR_DRIVER


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 (and as C++) on its own."""
    import shutil
    import subprocess
    src = tmp_path / "use_header.c"
    src.write_text('#include "symplex_b200.h"\nint main(void) { symplex_b200_comm c; symplex_gemm_desc d; (void)c; (void)d; return 0; }\n')
    inc = os.path.join(ROOT, "include")
    for cmd in (["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only"],
                ["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++"]):
        if shutil.which(cmd[0]) is None:
            pytest.skip(f"{cmd[0]} not installed")
        r = subprocess.run(cmd + ["-I", inc, str(src)], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
