"""Drop-in for the matmul / CUDA functions of the reference's pyo3 module ``symplex._symplex_core``
(``python/src/lib.rs``): same names, same raw-address arguments, same integer return convention.

Pointers are host addresses passed as Python ints (``arr.ctypes.data``), exactly as the reference's
callers do (``python/symplex/__init__.py:592``, ``bench_phase3_jit_vs_numpy.py:230``).
"""
from __future__ import annotations

import ctypes

from . import _capi


def parallel_matmul(a_ptr: int, b_ptr: int, c_ptr: int, m: int, n: int, k: int) -> int:
    """``python/src/lib.rs:1027-1039``: fp32 row-major C = A.B; returns 0 (zero dimension: no-op)."""
    return int(_capi.load().symplex_parallel_matmul(a_ptr, b_ptr, c_ptr, m, n, k))


def jit_parallel_matmul(a_ptr: int, b_ptr: int, c_ptr: int, m: int, n: int, k: int) -> int:
    """``python/src/lib.rs:1041-1062``."""
    return int(_capi.load().symplex_jit_parallel_matmul(a_ptr, b_ptr, c_ptr, m, n, k))


def cuda_matmul(a_ptr: int, b_ptr: int, c_ptr: int, m: int, n: int, k: int) -> int:
    """``python/src/lib.rs:1836-1849``: 0 on success, -1 on any CUDA error."""
    return int(_capi.load().symplex_cuda_matmul(a_ptr, b_ptr, c_ptr, m, n, k))


def cuda_available() -> bool:
    """``python/src/lib.rs:1713-1717``."""
    return bool(_capi.load().symplex_cuda_available())


def cuda_device_info() -> dict:
    """``python/src/lib.rs:1719-1753``: same keys; ``{"available": False, "error": ...}`` without a GPU."""
    lib = _capi.load()
    info = _capi.DeviceInfo()
    rc = lib.symplex_cuda_device_info(ctypes.byref(info))
    if rc != 0:
        return {"available": False, "error": _capi.last_error()}
    major, minor = info.compute_capability_major, info.compute_capability_minor
    return {
        "available": True,
        "name": info.name.decode("utf-8", "replace"),
        "sm_arch": f"sm_{major}{minor}",
        "compute_capability_major": major,
        "compute_capability_minor": minor,
        "total_memory_bytes": int(info.total_memory_bytes),
        "total_memory_gb": info.total_memory_bytes / 1e9,
        "num_sms": info.num_sms,
        "num_cuda_cores": info.num_cuda_cores,
        "warp_size": info.warp_size,
        "max_threads_per_block": info.max_threads_per_block,
        "max_shared_memory_per_block": info.max_shared_memory_per_block,
        "clock_mhz": info.clock_mhz,
    }


def cuda_info() -> str:
    """``python/src/lib.rs:1876-1880``: one-line human-readable description."""
    d = cuda_device_info()
    if not d["available"]:
        return f"CUDA not available: {d['error']}"
    return (f"{d['name']} ({d['sm_arch']}, {d['num_sms']} SMs, {d['total_memory_gb']:.1f} GB): "
            "symplex_b200 tcgen05 GEMM library")


def _simd_fused_elementwise(ops, input_ptrs, constants, n, reduce_op, dst_ptr, f64: bool) -> float:
    import math
    lib = _capi.load()
    arr = _capi.pack_fused_ops(ops)
    ptrs = (ctypes.c_void_p * max(len(input_ptrs), 1))(*[int(p) for p in input_ptrs])
    ctype = ctypes.c_double if f64 else ctypes.c_float
    consts = (ctype * max(len(constants), 1))(*[float(c) for c in constants])
    fn = lib.symplex_simd_fused_elementwise_f64 if f64 else lib.symplex_simd_fused_elementwise_f32
    v = fn(arr, len(ops), ptrs, len(input_ptrs), consts, len(constants), int(n), int(reduce_op),
           int(dst_ptr) if dst_ptr else None)
    if math.isnan(v) and _capi.last_error() != "no error":
        raise _capi.SymplexB200Error(_capi.ERR_EXEC, _capi.last_error())
    return float(v)


def simd_fused_elementwise_f32(ops, input_ptrs, constants, n: int, reduce_op: int, dst_ptr: int) -> float:
    """``python/src/lib.rs:1686-1695``: run a fused op chain over ``n`` elements of host ``float32`` arrays.

    ``ops`` is a list of ``(op, lhs_src, lhs_idx, rhs_src, rhs_idx)``; ``input_ptrs`` are host addresses as
    ints; ``reduce_op`` 0 / 1 / 2 returns the sum / max / min, 255 writes to ``dst_ptr`` and returns 0.0.
    One GPU pass per chunk of the arrays (single kernel: loads, the whole chain, store or reduction).
    """
    return _simd_fused_elementwise(ops, input_ptrs, constants, n, reduce_op, dst_ptr, False)


def simd_fused_elementwise_f64(ops, input_ptrs, constants, n: int, reduce_op: int, dst_ptr: int) -> float:
    """``python/src/lib.rs:1700-1709``: the same for ``float64`` arrays and constants."""
    return _simd_fused_elementwise(ops, input_ptrs, constants, n, reduce_op, dst_ptr, True)


def micro_kernel_config(target: str = "server", element_type: str = "fp32") -> dict:
    """``python/src/lib.rs:531-553``; target ``"b200"`` is added (see ``symplex_b200.planner``)."""
    from . import planner
    return planner.micro_kernel_config(target, element_type)


def cuda_compile_ptx(pattern_type: str, shape_info: dict, sm_arch: str = "sm_100a") -> str:
    """``python/src/lib.rs:1762-1832`` returns generated PTX text; this library runs precompiled kernels, so the
    string is a one-line description of the kernel that serves the pattern (``engine.cuda_compile_kernel``)."""
    from . import engine
    return engine.cuda_compile_kernel(pattern_type, shape_info, sm_arch).ptx_source()
