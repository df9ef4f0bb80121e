"""ctypes access to the CPU oracle (``oracle/liboracle.so``) and to the reference's own C kernels
compiled unchanged (``oracle/_ref/libsymplex_kernels.so``).

Test infrastructure only: imported by tests/, the smoke check and the benchmark's CPU-baseline leg,
never by the symplex_b200 package."""
import ctypes
import os
import subprocess

import numpy as np

ORACLE_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(ORACLE_DIR)
ORACLE_SO = os.path.join(ORACLE_DIR, "liboracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libsymplex_kernels.so")

_vp, _i64, _int, _f = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data)


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        for name in ("oracle_matmul_jit_order", "oracle_matmul_blis_order", "oracle_jit_parallel_matmul",
                     "oracle_parallel_matmul"):
            getattr(lib, name).argtypes = [_vp, _vp, _vp, _i64, _i64, _i64, _int]
            getattr(lib, name).restype = None
        for name in ("oracle_matmul_c_order", "oracle_scalar_matmul"):
            getattr(lib, name).argtypes = [_vp, _vp, _vp, _i64, _i64, _i64]
            getattr(lib, name).restype = None
        lib.oracle_fused_matmul_bias_relu.argtypes = [_vp, _vp, _vp, _i64, _i64, _i64, _vp]
        lib.oracle_fused_matmul_bias_relu.restype = None
        lib.oracle_bf16_round_array.argtypes = [_vp, _vp, _i64]
        lib.oracle_f32_to_bf16_bits.argtypes = [_vp, _vp, _i64]
        lib.oracle_bf16_bits_to_f32.argtypes = [_vp, _vp, _i64]
        lib.oracle_activation.argtypes = [_f, _int]
        lib.oracle_activation.restype = _f
        lib.oracle_epilogue.argtypes = [_vp, _i64, _i64, _f, _f, _vp, _vp, _int]
        lib.oracle_epilogue.restype = None
        lib.oracle_matmul_jit_order_rows.argtypes = [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int]
        lib.oracle_matmul_jit_order_rows.restype = None
        lib.oracle_max_threads.restype = _int
        lib.oracle_fused_elementwise_f32.argtypes = [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _int, _vp, _int]
        lib.oracle_fused_elementwise_f32.restype = ctypes.c_double
        lib.oracle_fused_elementwise_f64.argtypes = [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _int, _vp, _int]
        lib.oracle_fused_elementwise_f64.restype = ctypes.c_double
        lib.oracle_matmul_jit_avx512.argtypes = [_vp, _vp, _vp, _i64, _i64, _i64]
        lib.oracle_matmul_jit_avx512.restype = _int
        lib.oracle_cache_tiled_dgemm.argtypes = [_vp, _vp, _vp, _i64, _i64, _i64]
        lib.oracle_cache_tiled_dgemm.restype = None
        self.threads = max(1, int(lib.oracle_max_threads()))

    def matmul_jit_avx512(self, A, B):
        """The AVX-512 intrinsics twin of ``matmul_jit_order`` (one thread); None on a CPU without AVX-512F."""
        A, B = self._prep(A, B)
        C = np.full((A.shape[0], B.shape[1]), np.nan, np.float32)
        rc = self.lib.oracle_matmul_jit_avx512(_ptr(A), _ptr(B), _ptr(C), A.shape[0], B.shape[1], A.shape[1])
        return C if rc == 0 else None

    def cache_tiled_dgemm(self, A, B):
        """The reference's f64 tiled GEMM order (``rust-engine/src/phase3_jit.rs:578-650``)."""
        A = np.ascontiguousarray(A, dtype=np.float64)
        B = np.ascontiguousarray(B, dtype=np.float64)
        assert A.ndim == 2 and B.ndim == 2 and A.shape[1] == B.shape[0]
        C = np.full((A.shape[0], B.shape[1]), np.nan, np.float64)
        self.lib.oracle_cache_tiled_dgemm(_ptr(A), _ptr(B), _ptr(C), A.shape[0], B.shape[1], A.shape[1])
        return C

    def fused_elementwise(self, ops, inputs, constants, reduce_op=255, exact=False, dtype=np.float32):
        """The reference's fused op chain on host arrays: returns the result array (reduce_op 255) or the reduced
        value as the reference computes it (``exact=True``: the true max / min even when n % 8 != 0).
        ``dtype=np.float64`` selects the f64 twin."""
        rec = np.zeros(max(len(ops), 1), dtype=np.dtype([("op", "u1"), ("ls", "u1"), ("li", "<u2"), ("rs", "u1"),
                                                          ("pad", "u1"), ("ri", "<u2")]))
        for i, (op, ls, li, rs, ri) in enumerate(ops):
            rec[i] = (op, ls, li, rs, 0, ri)
        arrs = [np.ascontiguousarray(a, dtype=dtype).ravel() for a in inputs]
        n = arrs[0].size if arrs else 0
        ptrs = (ctypes.c_void_p * max(len(arrs), 1))(*[a.ctypes.data for a in arrs])
        consts = np.ascontiguousarray(np.asarray(list(constants) + [0.0], dtype=dtype))
        dst = np.zeros(n, dtype)
        fn = self.lib.oracle_fused_elementwise_f64 if dtype == np.float64 else self.lib.oracle_fused_elementwise_f32
        v = fn(_ptr(rec), len(ops), ctypes.cast(ptrs, _vp), len(arrs), _ptr(consts),
                                                  len(constants), n, int(reduce_op), _ptr(dst), int(bool(exact)))
        return dst if reduce_op == 255 else float(v)

    @staticmethod
    def _prep(A, B):
        A = np.ascontiguousarray(A, dtype=np.float32)
        B = np.ascontiguousarray(B, dtype=np.float32)
        assert A.ndim == 2 and B.ndim == 2 and A.shape[1] == B.shape[0]
        return A, B

    def _mm(self, fn, A, B, threads=None):
        A, B = self._prep(A, B)
        C = np.full((A.shape[0], B.shape[1]), np.nan, np.float32)
        fn(_ptr(A), _ptr(B), _ptr(C), A.shape[0], B.shape[1], A.shape[1], threads or self.threads)
        return C

    def matmul_jit_order(self, A, B, threads=None):
        return self._mm(self.lib.oracle_matmul_jit_order, A, B, threads)

    def matmul_blis_order(self, A, B, threads=None):
        return self._mm(self.lib.oracle_matmul_blis_order, A, B, threads)

    def jit_parallel_matmul(self, A, B, threads=None):
        """The reference's dispatcher on an AVX-512 host: JIT order for N >= 64, BLIS order otherwise."""
        return self._mm(self.lib.oracle_jit_parallel_matmul, A, B, threads)

    def matmul_c_order(self, A, B):
        A, B = self._prep(A, B)
        C = np.full((A.shape[0], B.shape[1]), np.nan, np.float32)
        self.lib.oracle_matmul_c_order(_ptr(A), _ptr(B), _ptr(C), A.shape[0], B.shape[1], A.shape[1])
        return C

    def scalar_matmul(self, A, B):
        A, B = self._prep(A, B)
        C = np.full((A.shape[0], B.shape[1]), np.nan, np.float32)
        self.lib.oracle_scalar_matmul(_ptr(A), _ptr(B), _ptr(C), A.shape[0], B.shape[1], A.shape[1])
        return C

    def fused_matmul_bias_relu(self, A, B, bias):
        A, B = self._prep(A, B)
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        C = np.full((A.shape[0], B.shape[1]), np.nan, np.float32)
        self.lib.oracle_fused_matmul_bias_relu(_ptr(A), _ptr(B), _ptr(C), A.shape[0], B.shape[1], A.shape[1],
                                               _ptr(bias))
        return C

    def matmul_rows(self, A, B, rows, threads=None):
        """Rows ``rows`` of A.B in JIT order (exact for a row-partitioned contraction)."""
        A, B = self._prep(A, B)
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        C = np.full((len(rows), B.shape[1]), np.nan, np.float32)
        self.lib.oracle_matmul_jit_order_rows(_ptr(A), _ptr(B), _ptr(C), _ptr(rows), len(rows), B.shape[1],
                                              A.shape[1], threads or self.threads)
        return C

    def bf16_round(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty_like(x)
        self.lib.oracle_bf16_round_array(_ptr(x), _ptr(out), x.size)
        return out

    def f32_to_bf16_bits(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.shape, np.uint16)
        self.lib.oracle_f32_to_bf16_bits(_ptr(x), _ptr(out), x.size)
        return out

    def bf16_bits_to_f32(self, bits):
        bits = np.ascontiguousarray(bits, dtype=np.uint16)
        out = np.empty(bits.shape, np.float32)
        self.lib.oracle_bf16_bits_to_f32(_ptr(bits), _ptr(out), bits.size)
        return out

    def activation(self, x, act):
        return np.array([self.lib.oracle_activation(float(v), act) for v in np.asarray(x).ravel()],
                        np.float32).reshape(np.shape(x))

    def epilogue(self, C, alpha=1.0, beta=0.0, residual=None, bias=None, act=0):
        """In-place act(alpha*C + beta*residual + bias) in fp32; returns C."""
        C = np.ascontiguousarray(C, dtype=np.float32)
        res = None if residual is None else np.ascontiguousarray(residual, dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self.lib.oracle_epilogue(_ptr(C), C.shape[0], C.shape[1], alpha, beta,
                                 _ptr(res) if res is not None else None, _ptr(b) if b is not None else None, act)
        return C


def load_oracle() -> Oracle:
    newest = max(os.path.getmtime(os.path.join(ORACLE_DIR, f)) for f in ("symplex_oracle.c", "symplex_oracle_avx512.c"))
    if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < newest:
        subprocess.run(["make", "-C", ORACLE_DIR, ORACLE_SO], check=True, capture_output=True)
    return Oracle(ctypes.CDLL(ORACLE_SO))


def load_ref_kernels():
    """The reference's kernels/matmul.c compiled unchanged, or None if it was never built here."""
    if not os.path.exists(REF_SO):
        return None
    lib = ctypes.CDLL(REF_SO)
    for name in ("symplex_matmul_f32", "symplex_matmul_tiled_f32"):
        getattr(lib, name).argtypes = [_vp, _vp, _vp, _i64, _i64, _i64]
        getattr(lib, name).restype = None
    return lib


def rel_frobenius(x, ref):
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = np.linalg.norm(ref)
    return float(np.linalg.norm(x - ref) / denom) if denom > 0 else float(np.linalg.norm(x))
