"""Drop-in for the matmul pyclasses of the reference's pyo3 module ``symplex_engine``
(``rust-engine/src/lib.rs:36-190``): kernel objects with ``execute_raw`` on raw host addresses.

The reference compiles x86 machine code in each constructor; here the "kernel" is the prebuilt
sm_100a library, so construction only checks that it can be loaded.
"""
from __future__ import annotations

from . import _capi
from .fusion import discover_fusions  # noqa: F401  (symplex_engine.discover_fusions, rust-engine/src/lib.rs:344-413)


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


class CudaGpuKernel:
    """``rust-engine/src/lib.rs:1405-1446``: what a "compiled" GPU kernel looks like to Python. This library ships
    precompiled sm_100a kernels, so ``ptx_source()`` is a one-line description rather than PTX text and
    ``ptx_size()`` is its length; the launch geometry and the estimate are the real ones."""

    def __init__(self, description, name, gflops, grid, block, smem):
        self._d, self._name, self._gflops, self._grid, self._block, self._smem = description, name, gflops, grid, block, smem

    def ptx_source(self) -> str:
        return self._d

    def kernel_name(self) -> str:
        return self._name

    def ptx_size(self) -> int:
        return len(self._d)

    def estimated_gflops(self) -> float:
        return self._gflops

    def grid_dims(self):
        return self._grid

    def block_dims(self):
        return self._block

    def shared_mem_bytes(self) -> int:
        return self._smem


def cuda_compile_kernel(pattern_type: str, shape_info: dict, sm_arch: str = "sm_100a") -> CudaGpuKernel:
    """``rust-engine/src/lib.rs:1500-1573``: describe the kernel that serves a pattern. ``"matmul"`` takes
    ``M, N, K`` (tile hints are accepted and ignored: the library picks the tile); ``"elementwise"`` takes
    ``op, n``; ``"fma"`` takes ``n``; ``"reduction"`` takes ``op`` (add / max / min) and ``n``. Unknown patterns and
    ops raise ``ValueError`` like the reference; ``"stencil"`` is not part of this library."""
    import ctypes
    from . import planner
    if pattern_type == "matmul":
        m, n, k = int(shape_info["M"]), int(shape_info["N"]), int(shape_info["K"])
        r = planner.compile_matmul(m, n, k, dtype="fp32")
        if not r.valid:
            raise ValueError(r.error)
        text = (f"// precompiled {sm_arch} kernel {r.kernel_name}: tile {r.optimal_tile}, tcgen05.mma {r.mma_shape}, "
                f"{r.stages} stages, {r.tmem_columns} TMEM columns")
        return CudaGpuKernel(text, r.kernel_name, r.estimated_tflops * 1e3, r.grid_dims, r.block_dims, r.shared_mem_bytes)
    if pattern_type in ("elementwise", "fma", "reduction"):
        if pattern_type == "elementwise" and shape_info["op"] not in _BINOPS:
            raise ValueError(f"Unsupported elementwise op: {shape_info['op']}")
        if pattern_type == "reduction" and shape_info["op"] not in ("add", "max", "min"):
            raise ValueError(f"Unsupported reduction op: {shape_info['op']}")
        n = int(shape_info["n"])
        n_in = {"elementwise": 2, "fma": 3, "reduction": 1}[pattern_type]
        streams = n_in + (0 if pattern_type == "reduction" else 1)
        grid, block, smem = (ctypes.c_int32 * 3)(), (ctypes.c_int32 * 3)(), ctypes.c_int32(0)
        _capi.check(_capi.load().symplex_b200_fused_elementwise_plan(n_in, n, 4, 0, ctypes.byref(grid), ctypes.byref(block),
                                                                     ctypes.byref(smem)))
        t = planner.hardware_target()
        seconds = 4.0 * streams * n / (t["global_bw_gbps"] * 1e9) + 4e-6
        flops = {"elementwise": 1, "fma": 2, "reduction": 1}[pattern_type] * n
        text = (f"// precompiled {sm_arch} kernel fused_elementwise_ring_kernel: {pattern_type}, {n_in} input array(s), "
                f"{streams} HBM stream(s)")
        return CudaGpuKernel(text, "fused_elementwise_ring_kernel", flops / seconds / 1e9, tuple(grid), tuple(block),
                             int(smem.value))
    raise ValueError(f"Unknown pattern type: {pattern_type}. Supported: matmul, elementwise, fma, reduction")
