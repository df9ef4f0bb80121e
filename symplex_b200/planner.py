"""Planning-side mirror of the reference for the matmul path: what the hardware is, which kernel a problem
gets and what it should cost. Host-only (no GPU needed); every answer comes from ``libsymplex_b200.so`` so it
cannot drift from what the launch path does.

* ``hardware_target()``          — ``hardware::HardwareTarget::B200()`` (``include/symplex/hardware/hardware_target.h:303-329``)
* ``micro_kernel_config()``      — ``_symplex_core.micro_kernel_config`` (``python/src/lib.rs:531-553``) /
                                   ``poly_get_micro_kernel_config`` (``rust-engine/src/ffi.rs:695-717``), plus target ``"b200"``
* ``compile_matmul()``           — ``training::CompilerPipeline::compile_matmul`` -> ``PipelineResult``
                                   (``include/symplex/training/compiler_pipeline.h:18-33,70``)
* ``LaunchConfig``               — ``cuda_backend::LaunchConfig`` (``rust-engine/src/cuda_backend.rs:123-155``)
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Tuple

from . import _capi

_TARGETS = {"server": 0, "edge": 1, "tensor": 2, "b200": 3}
_ELEMENT_BYTES = {"fp64": 8, "fp32": 4, "fp16": 2, "bf16": 2, "int8": 1, "int4": 1}


def hardware_target() -> dict:
    """The B200 as this library's kernels see it (148 SMs, tcgen05 atom, measured and nominal peaks)."""
    t = _capi.Target()
    _capi.check(_capi.load().symplex_b200_hardware_target(ctypes.byref(t)))
    out = {name: getattr(t, name) for name, _ in _capi.Target._fields_}
    out["mma_dtype"] = t.mma_dtype.decode()
    return out


def micro_kernel_config(target: str = "server", element_type: str = "fp32") -> dict:
    """Tile configuration for a target. Unknown targets fall back to ``"server"`` and unknown element types to
    fp32, as the reference's ``parse_target`` / ``parse_element_type`` do (``python/src/lib.rs:66-84``)."""
    code = _TARGETS.get(target, 0)
    ebytes = _ELEMENT_BYTES.get(element_type, 4)
    vals = [ctypes.c_size_t(0) for _ in range(5)]
    _capi.load().symplex_b200_micro_kernel_config(code, ebytes, *[ctypes.byref(v) for v in vals])
    m, n, k, acc, pf = (int(v.value) for v in vals)
    if code == 3:
        buffers = pf + 1
    elif code == 1:
        buffers = 1
    else:
        buffers = 2
    return {"tile_m": m, "tile_n": n, "tile_k": k, "accumulator_registers": acc, "prefetch_distance": pf,
            "double_buffer_count": buffers}


@dataclass
class LaunchConfig:
    """Grid, block and shared memory of one launch."""
    grid: Tuple[int, int, int]
    block: Tuple[int, int, int]
    shared_mem_bytes: int

    @staticmethod
    def elementwise(n: int, threads_per_block: int) -> "LaunchConfig":
        """``LaunchConfig::elementwise`` (``cuda_backend.rs:134-141``): one thread per element."""
        return LaunchConfig(((n + threads_per_block - 1) // threads_per_block, 1, 1), (threads_per_block, 1, 1), 0)

    @staticmethod
    def matmul(m: int, n: int, tile_m: int, tile_n: int) -> "LaunchConfig":
        """``LaunchConfig::matmul`` (``cuda_backend.rs:144-154``): the reference's one-warp-per-tile geometry,
        kept for callers that ask for it by tile size. What this library launches is ``compile_matmul().launch``."""
        return LaunchConfig(((n + tile_n - 1) // tile_n, (m + tile_m - 1) // tile_m, 1), (32, 1, 1),
                            tile_m * tile_n * 4 * 2)


@dataclass
class PipelineResult:
    """Fields of the reference's ``PipelineResult`` that apply to precompiled kernels (no ``ptx_source``)."""
    kernel_name: str
    optimal_tile: Tuple[int, int, int]
    mma_shape: Tuple[int, int, int]
    estimated_latency_ns: float
    estimated_tflops: float
    speedup_vs_naive: float
    grid_dims: Tuple[int, int, int]
    block_dims: Tuple[int, int, int]
    cluster_size: int
    stages: int
    shared_mem_bytes: int
    tmem_columns: int
    prepass_launches: int
    workspace_bytes: int
    tiles: int
    flops: float
    bytes: float
    bound: str
    valid: bool
    error: str

    @property
    def launch(self) -> LaunchConfig:
        return LaunchConfig(self.grid_dims, self.block_dims, self.shared_mem_bytes)


def compile_matmul(M: int, N: int, K: int, *, dtype: str = "bf16", out_dtype: str | None = None, batch: int = 1,
                   b_layout: int = _capi.ROW_MAJOR, activation=None, num_sms: int = 0) -> PipelineResult:
    """Which kernel ``symplex_b200_gemm`` would launch for this problem, and its estimated cost.

    Like the reference, failure is reported in the result (``valid`` False, ``error`` set), not raised."""
    dts = {"bf16": _capi.DT_BF16, "fp32": _capi.DT_F32, "f32": _capi.DT_F32}
    lib = _capi.load()
    d = _capi.GemmDesc()
    in_dt = dts.get(dtype, -1)
    lib.symplex_b200_gemm_desc_init(ctypes.byref(d), M, N, K, in_dt, dts.get(out_dtype or dtype, -1))
    d.batch = batch
    d.b_layout = b_layout
    d.activation = _capi.ACTIVATIONS.get(activation, -1) if (activation is None or isinstance(activation, str)) \
        else int(activation)
    p = _capi.GemmPlan()
    lib.symplex_b200_gemm_plan(ctypes.byref(d), num_sms, ctypes.byref(p))
    return PipelineResult(
        kernel_name=p.kernel_name.decode(), optimal_tile=(p.tile_m, p.tile_n, p.tile_k),
        mma_shape=(p.mma_m, p.mma_n, p.mma_k), estimated_latency_ns=p.estimated_latency_ns,
        estimated_tflops=p.estimated_tflops, speedup_vs_naive=p.speedup_vs_naive, grid_dims=tuple(p.grid_dims),
        block_dims=tuple(p.block_dims), cluster_size=p.cluster_size, stages=p.stages,
        shared_mem_bytes=p.shared_mem_bytes, tmem_columns=p.tmem_columns, prepass_launches=p.prepass_launches,
        workspace_bytes=int(p.workspace_bytes), tiles=int(p.tiles), flops=p.flops, bytes=p.bytes,
        bound="hbm" if p.bound == 1 else "tensor", valid=bool(p.valid), error=p.error.decode())
