"""ctypes binding of ``libsymplex_b200.so`` (declarations: ``include/symplex_b200.h``).

The shared library is the product; this module only loads it and describes its C ABI to Python.
There is no fallback: if the library is missing, ``load()`` raises with the build command.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (c_char, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_size_t, c_uint8, c_uint16, c_uint64,
                    c_void_p)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsymplex_b200.so")

OK, ERR_DRIVER, ERR_INVALID, ERR_OOM, ERR_EXEC, ERR_TIMEOUT = 0, -1, -2, -3, -4, -5
DT_F32, DT_BF16 = 9, 11
ROW_MAJOR, COL_MAJOR = 0, 1
ACT_NONE, ACT_RELU, ACT_GELU, ACT_SIGMOID, ACT_TANH, ACT_SILU = range(6)
ACTIVATIONS = {
    None: ACT_NONE, "none": ACT_NONE, "relu": ACT_RELU, "gelu": ACT_GELU,
    "sigmoid": ACT_SIGMOID, "tanh": ACT_TANH, "silu": ACT_SILU,
}


class GemmDesc(ctypes.Structure):
    """``symplex_gemm_desc``."""
    _fields_ = [
        ("M", c_int64), ("N", c_int64), ("K", c_int64),
        ("batch", c_int32), ("in_dtype", c_int32), ("out_dtype", c_int32), ("b_layout", c_int32),
        ("lda", c_int64), ("ldb", c_int64), ("ldc", c_int64),
        ("a_batch_stride", c_int64), ("b_batch_stride", c_int64), ("c_batch_stride", c_int64),
        ("alpha", c_float), ("beta", c_float),
        ("activation", c_int32), ("tile_n", c_int32),
    ]


class DeviceInfo(ctypes.Structure):
    """``symplex_device_info``."""
    _fields_ = [
        ("name", c_char * 256),
        ("compute_capability_major", c_int32), ("compute_capability_minor", c_int32),
        ("total_memory_bytes", c_uint64),
        ("num_sms", c_int32), ("num_cuda_cores", c_int32), ("warp_size", c_int32),
        ("max_threads_per_block", c_int32), ("max_shared_memory_per_block", c_int32),
        ("clock_mhz", c_int32),
    ]


class FusedOp(ctypes.Structure):
    """``symplex_fused_op`` (the reference's ``FusedOpDesc``, 8 bytes)."""
    _fields_ = [("op", c_uint8), ("lhs_src", c_uint8), ("lhs_idx", c_uint16), ("rhs_src", c_uint8),
                ("reserved", c_uint8), ("rhs_idx", c_uint16)]


class KernelArgs(ctypes.Structure):
    """``symplex_kernel_args`` (the reference's ``jit::KernelArgs``)."""
    _fields_ = [("data", c_void_p), ("data_size", c_int64), ("input_ptrs", ctypes.POINTER(c_void_p)),
                ("num_inputs", c_int64), ("input_sizes", ctypes.POINTER(c_int64)),
                ("M", c_int64), ("N", c_int64), ("K", c_int64), ("batch", c_int64)]


class Target(ctypes.Structure):
    """``symplex_b200_target``."""
    _fields_ = [
        ("num_sms", c_int32), ("warp_size", c_int32), ("max_warps_per_sm", c_int32), ("max_threads_per_sm", c_int32),
        ("shared_mem_bytes_per_sm", c_int32), ("max_shared_mem_per_block", c_int32),
        ("register_file_bytes_per_sm", c_int32), ("tensor_memory_bytes_per_sm", c_int32),
        ("max_registers_per_thread", c_int32), ("num_fp32_lanes_per_sm", c_int32),
        ("mma_m", c_int32), ("mma_n", c_int32), ("mma_k", c_int32), ("mma_pair_m", c_int32),
        ("mma_dtype", c_char * 8),
        ("global_bw_gbps", c_double), ("global_bw_nominal_gbps", c_double),
        ("bf16_dense_tflops", c_double), ("bf16_dense_tflops_sustained", c_double),
        ("bf16_dense_tflops_nominal", c_double), ("global_capacity_gb", c_double),
        ("l2_cache_kb", c_int32), ("nvlink_gbps_per_direction", c_double),
        ("has_tma", c_int32), ("has_async_copy", c_int32), ("has_tensor_memory", c_int32),
        ("pipeline_stages", c_int32), ("from_device", c_int32),
    ]


class GemmPlan(ctypes.Structure):
    """``symplex_gemm_plan``."""
    _fields_ = [
        ("kernel_name", c_char * 64),
        ("tile_m", c_int32), ("tile_n", c_int32), ("tile_k", c_int32),
        ("mma_m", c_int32), ("mma_n", c_int32), ("mma_k", c_int32),
        ("cluster_size", c_int32), ("stages", c_int32),
        ("grid_dims", c_int32 * 3), ("block_dims", c_int32 * 3),
        ("shared_mem_bytes", c_int32), ("tmem_columns", c_int32),
        ("prepass_launches", c_int32), ("bound", c_int32),
        ("tiles", c_int64), ("workspace_bytes", c_size_t),
        ("flops", c_double), ("bytes", c_double),
        ("estimated_latency_ns", c_double), ("estimated_tflops", c_double), ("speedup_vs_naive", c_double),
        ("valid", c_int32), ("error", c_char * 128),
    ]


class Comm(ctypes.Structure):
    """``symplex_b200_comm``."""
    _fields_ = [("rank", c_int32), ("world", c_int32), ("c_base", c_void_p * 8), ("c_multicast", c_void_p),
                ("flags", c_void_p * 8), ("epoch", c_int64), ("wait_limit_ms", c_int32), ("reserved", c_int32)]


class ShardSpec(ctypes.Structure):
    """``symplex_shard_spec``."""
    _fields_ = [("strategy", c_int32), ("shard_dim", c_int32), ("original_shape", c_int64 * 2),
                ("local_shape", c_int64 * 2)]


class ShardPlanPOD(ctypes.Structure):
    """``symplex_shard_plan``."""
    _fields_ = [("a", ShardSpec), ("b", ShardSpec), ("c", ShardSpec),
                ("n_all_gather_ops", c_int32), ("n_all_reduce_ops", c_int32), ("n_all_to_all_ops", c_int32),
                ("world", c_int32), ("total_communication_bytes", c_int64), ("peak_memory_per_device", c_int64)]


class GeneratedKernel(ctypes.Structure):
    """``symplex_generated_kernel``."""
    _fields_ = [("kernel_name", c_char * 64), ("shared_mem_bytes", c_int64), ("register_count", c_int64),
                ("grid_dims", c_int64 * 3), ("block_dims", c_int64 * 3), ("valid", c_int32),
                ("error_message", c_char * 128)]


class FusionOp(ctypes.Structure):
    """``symplex_fusion_op``."""
    _fields_ = [("op", c_char_p), ("shape", ctypes.POINTER(c_int64)), ("rank", c_int32), ("dtype", c_char_p)]


XCHG_AUTO, XCHG_UNICAST, XCHG_MULTICAST, XCHG_EPILOGUE_TMA = 0, 1, 2, 3
COMM_FLAG_WORDS = 16
DT_F64 = 10

REDUCE_SUM, REDUCE_MAX, REDUCE_MIN, REDUCE_NONE = 0, 1, 2, 255

_F32P = c_void_p  # raw addresses; callers pass ints (numpy ``.ctypes.data`` / torch ``.data_ptr()``)

# name -> (restype, argtypes): every symbol include/symplex_b200.h declares.
SIGNATURES = {
    "symplex_b200_gemm_desc_init": (None, [ctypes.POINTER(GemmDesc), c_int64, c_int64, c_int64, c_int32, c_int32]),
    "symplex_b200_gemm_workspace_bytes": (c_size_t, [ctypes.POINTER(GemmDesc)]),
    "symplex_b200_gemm": (c_int, [ctypes.POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "symplex_b200_gemm_peers": (c_int, [ctypes.POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        ctypes.POINTER(c_void_p), c_int32, c_void_p]),
    "symplex_b200_gemm_ws": (c_int, [ctypes.POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_size_t, c_void_p]),
    "symplex_b200_sgemm_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "symplex_b200_sharded_gemm": (c_int, [ctypes.POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, ctypes.POINTER(Comm),
                                          c_int32, c_void_p]),
    "symplex_b200_analyze_matmul": (c_int, [c_int64, c_int64, c_int64, c_int32, c_int32, ctypes.POINTER(ShardPlanPOD)]),
    "symplex_b200_noalloc_status": (c_int, [c_void_p]),
    "symplex_b200_selftest_wait_timeout": (c_int, [c_void_p, c_void_p, c_void_p, c_int32, c_void_p]),
    "symplex_b200_set_option": (c_int, [c_char_p, c_int64]),
    "symplex_b200_get_option": (c_int64, [c_char_p]),
    "symplex_b200_stream_k_items": (c_int32, [c_int32, c_int32, c_int32, c_int32, ctypes.POINTER(c_int32), c_int32,
                                              ctypes.POINTER(c_int32)]),
    "blas_dgemm": (None, [_F32P, _F32P, _F32P, c_size_t, c_size_t, c_size_t]),
    "cache_tiled_dgemm_thin": (None, [_F32P, _F32P, _F32P, c_size_t, c_size_t, c_size_t]),
    "symplex_b200_dgemm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                   c_void_p]),
    "poly_get_micro_kernel_config": (None, [c_uint8, c_size_t] + [ctypes.POINTER(c_size_t)] * 5),
    "symplex_b200_generate_matmul": (c_int, [c_int64, c_int64, c_int64, c_int32, c_int64, c_int64, c_int64,
                                             ctypes.POINTER(GeneratedKernel)]),
    "symplex_b200_discover_fusions": (c_int64, [ctypes.POINTER(FusionOp), c_size_t, c_char_p, c_size_t]),
    "symplex_b200_compile_epilogue": (c_int, [ctypes.POINTER(FusionOp), c_size_t, c_size_t, ctypes.POINTER(GemmDesc),
                                              ctypes.POINTER(c_int32), ctypes.POINTER(c_int32),
                                              ctypes.POINTER(c_int32)]),
    "symplex_b200_abi_sizes_ext": (c_int32, [ctypes.POINTER(c_int32), c_int32]),
    "symplex_b200_sync_status": (c_int, [c_void_p]),
    "symplex_b200_last_error": (c_char_p, []),
    "symplex_b200_gemm_host": (c_int, [ctypes.POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "symplex_cuda_matmul": (c_int64, [_F32P, _F32P, _F32P, c_int64, c_int64, c_int64]),
    "symplex_parallel_matmul": (c_int64, [_F32P, _F32P, _F32P, c_int64, c_int64, c_int64]),
    "symplex_jit_parallel_matmul": (c_int64, [_F32P, _F32P, _F32P, c_int64, c_int64, c_int64]),
    "symplex_exec_matmul": (c_int64, [_F32P, _F32P, _F32P, c_int64, c_int64, c_int64]),
    "symplex_exec_fused_matmul_bias_relu": (c_int64, [_F32P, _F32P, _F32P, c_int64, c_int64, c_int64, _F32P]),
    "symplex_matmul_f32": (None, [_F32P, _F32P, _F32P, c_int64, c_int64, c_int64]),
    "symplex_matmul_tiled_f32": (None, [_F32P, _F32P, _F32P, c_int64, c_int64, c_int64]),
    "blas_sgemm": (None, [_F32P, _F32P, _F32P, c_size_t, c_size_t, c_size_t]),
    "cache_tiled_sgemm_thin": (None, [_F32P, _F32P, _F32P, c_size_t, c_size_t, c_size_t]),
    "symplex_b200_exec_tensor_matmul": (c_int64, [c_char_p, c_size_t, ctypes.POINTER(c_void_p), c_size_t]),
    "symplex_b200_execute": (c_int, [c_char_p, ctypes.POINTER(KernelArgs)]),
    "symplex_cuda_available": (c_int, []),
    "symplex_cuda_device_info": (c_int, [ctypes.POINTER(DeviceInfo)]),
    "symplex_b200_launch_count": (c_uint64, []),
    "symplex_b200_abi_sizes": (None, [ctypes.POINTER(c_int32 * 5)]),
    "symplex_simd_fused_elementwise_f32": (c_double, [ctypes.POINTER(FusedOp), c_size_t, ctypes.POINTER(c_void_p), c_size_t,
                                                      ctypes.POINTER(c_float), c_size_t, c_size_t, c_uint8, _F32P]),
    "symplex_simd_fused_elementwise_f64": (c_double, [ctypes.POINTER(FusedOp), c_size_t, ctypes.POINTER(c_void_p), c_size_t,
                                                      ctypes.POINTER(c_double), c_size_t, c_size_t, c_uint8, _F32P]),
    "symplex_b200_fused_elementwise_f64": (c_int, [ctypes.POINTER(FusedOp), c_size_t, ctypes.POINTER(c_void_p), c_size_t,
                                                   ctypes.POINTER(c_double), c_size_t, c_int64, c_int, _F32P, c_void_p,
                                                   c_void_p]),
    "symplex_b200_fused_elementwise_f32": (c_int, [ctypes.POINTER(FusedOp), c_size_t, ctypes.POINTER(c_void_p), c_size_t,
                                                   ctypes.POINTER(c_float), c_size_t, c_int64, c_int, _F32P, c_void_p,
                                                   c_void_p]),
    "symplex_cuda_elementwise": (c_int64, [_F32P, _F32P, _F32P, c_int64, c_int]),
    "symplex_b200_fused_program_info": (c_int, [ctypes.POINTER(FusedOp), c_size_t, c_size_t, ctypes.POINTER(c_int),
                                                ctypes.POINTER(c_int)]),
    "symplex_b200_fused_elementwise_plan": (c_int, [c_int, c_int64, c_int, c_int, ctypes.POINTER(c_int32 * 3),
                                                    ctypes.POINTER(c_int32 * 3), ctypes.POINTER(c_int32)]),
    "symplex_b200_hardware_target": (c_int, [ctypes.POINTER(Target)]),
    "symplex_b200_micro_kernel_config": (None, [c_uint8, c_size_t] + [ctypes.POINTER(c_size_t)] * 5),
    "symplex_b200_gemm_plan": (c_int, [ctypes.POINTER(GemmDesc), c_int, ctypes.POINTER(GemmPlan)]),
}


def pack_fused_ops(ops):
    """``[(op, lhs_src, lhs_idx, rhs_src, rhs_idx), ...]`` -> a ctypes array of ``FusedOp``."""
    arr = (FusedOp * max(len(ops), 1))()
    for i, (op, ls, li, rs, ri) in enumerate(ops):
        arr[i] = FusedOp(int(op), int(ls), int(li), int(rs), 0, int(ri))
    return arr

_lib = None


class SymplexB200Error(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"symplex_b200 error {code}: {message}")
        self.code = code


def load() -> ctypes.CDLL:
    """Load the library (once) and attach the signatures. Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m symplex_b200.build` "
            "(nvcc, sm_100a). There is no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library out of sync
        fn.restype = restype
        fn.argtypes = argtypes
    sizes = (c_int32 * 10)()
    lib.symplex_b200_abi_sizes_ext(sizes, 10)
    mine = [ctypes.sizeof(t) for t in (GemmDesc, DeviceInfo, FusedOp, Target, GemmPlan, Comm, ShardPlanPOD,
                                       GeneratedKernel, FusionOp, KernelArgs)]
    if list(sizes) != mine:
        raise ImportError(f"struct layouts of {LIB_PATH} {list(sizes)} differ from this binding's {mine}: rebuild")
    _lib = lib
    return lib


def pack_fusion_ops(ops):
    """``[(name, shape, dtype), ...]`` -> (ctypes array of ``FusionOp``, keep-alive list)."""
    arr = (FusionOp * max(len(ops), 1))()
    keep = []
    for i, (name, shape, dtype) in enumerate(ops):
        sh = (c_int64 * max(len(shape), 1))(*[int(x) for x in shape])
        keep.append(sh)
        arr[i] = FusionOp(str(name).encode(), ctypes.cast(sh, ctypes.POINTER(c_int64)), len(shape), str(dtype).encode())
    return arr, keep


class option:
    """``with option("pair_mode", 1): ...`` - set a tuning override of the library, restore it afterwards."""

    def __init__(self, name: str, value: int):
        self.name, self.value = name.encode(), int(value)

    def __enter__(self):
        lib = load()
        self.old = lib.symplex_b200_get_option(self.name)
        check(lib.symplex_b200_set_option(self.name, self.value))
        return self

    def __exit__(self, *exc):
        load().symplex_b200_set_option(self.name, self.old)
        return False


def last_error() -> str:
    return load().symplex_b200_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    if code != 0:
        raise SymplexB200Error(int(code), last_error())
