"""Drop-in for the matmul pyclasses of the reference's pyo3 module ``symplex_engine``
(``rust-engine/src/lib.rs:36-190``): kernel objects with ``execute_raw`` on raw host addresses.

The reference compiles x86 machine code in each constructor; here the "kernel" is the prebuilt
sm_100a library, so construction only checks that it can be loaded.
"""
from __future__ import annotations

from . import _capi


class _KernelBase:
    _isa = "sm_100a"

    def __init__(self):
        try:
            self._lib = _capi.load()
        except (ImportError, OSError) as e:  # the reference raises PyRuntimeError when compilation fails
            raise RuntimeError(f"Failed to load matmul kernel library: {e}") from e

    def isa_level(self) -> str:
        return self._isa


class MatmulKernel(_KernelBase):
    """``rust-engine/src/lib.rs:43-78``."""

    def execute_raw(self, a_ptr: int, b_ptr: int, c_ptr: int, m: int, n: int, k: int) -> int:
        return int(self._lib.symplex_exec_matmul(a_ptr, b_ptr, c_ptr, m, n, k))


class AVX2MatmulKernel(MatmulKernel):
    """``rust-engine/src/lib.rs:80-113``."""


class AVX512MatmulKernel(_KernelBase):
    """``rust-engine/src/lib.rs:115-160``: dimensions are fixed at construction; ``execute_raw`` ignores
    the dimensions passed to it and uses the constructor's, as the reference does (:144-153)."""

    def __init__(self, m: int, n: int, k: int):
        if m == 0 or n == 0 or k == 0:
            raise ValueError("AVX512MatmulKernel dimensions must be non-zero")
        super().__init__()
        self._dims = (int(m), int(n), int(k))

    def execute_raw(self, a_ptr: int, b_ptr: int, c_ptr: int, _m: int = 0, _n: int = 0, _k: int = 0) -> int:
        m, n, k = self._dims
        return int(self._lib.symplex_exec_matmul(a_ptr, b_ptr, c_ptr, m, n, k))

    def dims(self):
        return self._dims


class FusedMatMulBiasReLUKernel(_KernelBase):
    """``rust-engine/src/lib.rs:160-190``: note the argument order — ``bias_ptr`` comes before m, n, k."""

    def execute_raw(self, a_ptr: int, b_ptr: int, c_ptr: int, bias_ptr: int, m: int, n: int, k: int) -> int:
        return int(self._lib.symplex_exec_fused_matmul_bias_relu(a_ptr, b_ptr, c_ptr, m, n, k, bias_ptr))


def cuda_matmul_raw(a_ptr: int, b_ptr: int, c_ptr: int, m: int, n: int, k: int) -> int:
    """``rust-engine/src/lib.rs:1589-1592``: 0 or -1."""
    return int(_capi.load().symplex_cuda_matmul(a_ptr, b_ptr, c_ptr, m, n, k))


_BINOPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "min": 4, "max": 5}


def cuda_elementwise_raw(a_ptr: int, b_ptr: int, dst_ptr: int, n: int, op: str) -> int:
    """``rust-engine/src/lib.rs:1597-1626``: ``dst = a <op> b`` on host float32 arrays; 0, -1 (CUDA error)
    or -2 (unknown op)."""
    if n == 0:
        return 0
    code = _BINOPS.get(op)
    if code is None:
        return -2
    return int(_capi.load().symplex_cuda_elementwise(a_ptr, b_ptr, dst_ptr, n, code))
