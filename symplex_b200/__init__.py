"""symplex_b200 — SympleX's dense-matmul hot path on B200 (sm_100a).

Host-side mirror of the reference's Python surface for this path. All arithmetic happens in
``libsymplex_b200.so`` (hand-written CUDA, C ABI in ``include/symplex_b200.h``); this package only
validates arguments the way the reference does and forwards raw addresses.

* ``matmul_jit`` / ``matmul_tiled``          — ``python/symplex/__init__.py:562-634`` of the reference
* ``_symplex_core`` (sub-module)             — the pyo3 functions of ``python/src/lib.rs`` for this path
* ``engine`` (sub-module)                    — the pyclasses of ``rust-engine/src/lib.rs`` for this path
* ``gemm`` / ``gemm_host``                   — the general fused GEMM (bf16 or fp32 inputs, epilogues)
* ``sharding`` (sub-module)                  — ShardPlan vocabulary + the row-sharded multi-GPU GEMM

There is no CPU fallback: every compute call raises (or returns the reference's error code) when the
library or a B200 is missing.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _capi
from ._capi import (ACT_GELU, ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SILU, ACT_TANH, ACTIVATIONS, COL_MAJOR, DT_BF16,
                    DT_F32, ROW_MAJOR, GemmDesc, SymplexB200Error)

__all__ = [
    "matmul_jit", "matmul_tiled", "matmul", "fused_matmul_bias_relu", "gemm", "gemm_host", "make_desc",
    "cuda_available", "launch_count", "SymplexB200Error", "fused_elementwise",
]


def make_desc(M, N, K, in_dtype=DT_F32, out_dtype=DT_F32, *, batch=1, b_layout=ROW_MAJOR, alpha=1.0, beta=0.0,
              activation=None, tile_n=0, lda=0, ldb=0, ldc=0) -> GemmDesc:
    """Build a ``symplex_gemm_desc``. ``activation`` is a name (``"gelu"``...) or a ``ACT_*`` code."""
    lib = _capi.load()
    d = GemmDesc()
    lib.symplex_b200_gemm_desc_init(ctypes.byref(d), M, N, K, in_dtype, out_dtype)
    d.batch = batch
    d.b_layout = b_layout
    d.alpha = alpha
    d.beta = beta
    if isinstance(activation, str) or activation is None:
        if activation not in ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; expected one of {sorted(k for k in ACTIVATIONS if k)}")
        d.activation = ACTIVATIONS[activation]
    else:
        d.activation = int(activation)
    d.tile_n = tile_n
    d.lda, d.ldb, d.ldc = lda, ldb, ldc
    return d


def cuda_available() -> bool:
    return bool(_capi.load().symplex_cuda_available())


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(_capi.load().symplex_b200_launch_count())


# ----------------------------------------------------------------------------- reference-shaped API

def _as_f32_2d(A, B, who):
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    if A.ndim != 2 or B.ndim != 2:
        raise ValueError(f"{who} requires 2D arrays")
    if A.shape[1] != B.shape[0]:
        raise ValueError(f"Shape mismatch: A is {A.shape}, B is {B.shape}")
    return A, B


def matmul_jit(A, B) -> np.ndarray:
    """``symplex.matmul_jit`` (``python/symplex/__init__.py:562-611``): fp32 ``A @ B`` for 2-D arrays.

    Same argument handling and ``ValueError``s as the reference; the product itself runs on the GPU
    through ``symplex_jit_parallel_matmul`` (3xTF32 on tensor cores, fp32-level accuracy).
    """
    A, B = _as_f32_2d(A, B, "matmul_jit")
    M, K = A.shape
    N = B.shape[1]
    C = np.zeros((M, N), dtype=np.float32)
    rc = _capi.load().symplex_jit_parallel_matmul(A.ctypes.data, B.ctypes.data, C.ctypes.data, M, N, K)
    _capi.check(rc)
    return C


def matmul_tiled(A, B) -> np.ndarray:
    """``symplex.matmul_tiled`` (``python/symplex/__init__.py:614-634``), same contract as ``matmul_jit``."""
    A, B = _as_f32_2d(A, B, "matmul_tiled")
    M, K = A.shape
    N = B.shape[1]
    C = np.zeros((M, N), dtype=np.float32)
    lib = _capi.load()
    lib.symplex_matmul_tiled_f32(A.ctypes.data, B.ctypes.data, C.ctypes.data, M, N, K)
    # The C entry point has no return value; after a failure it has filled C with NaN and left the reason.
    if M and N and _capi.last_error() != "no error":
        raise SymplexB200Error(_capi.ERR_EXEC if lib.symplex_cuda_available() else _capi.ERR_DRIVER, _capi.last_error())
    return C


matmul = matmul_jit


def fused_matmul_bias_relu(A, B, bias) -> np.ndarray:
    """``max(A @ B + bias, 0)`` — the reference's one executed fused kernel
    (``rust-engine/src/x86_emitter.rs:634-770``), as a single GPU kernel with a fused epilogue."""
    A, B = _as_f32_2d(A, B, "fused_matmul_bias_relu")
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    M, K = A.shape
    N = B.shape[1]
    if bias.shape != (N,):
        raise ValueError(f"bias must have shape ({N},), got {bias.shape}")
    C = np.zeros((M, N), dtype=np.float32)
    rc = _capi.load().symplex_exec_fused_matmul_bias_relu(A.ctypes.data, B.ctypes.data, C.ctypes.data, M, N, K,
                                                          bias.ctypes.data)
    _capi.check(rc)
    return C


# ----------------------------------------------------------------------------- general fused GEMM

def gemm_host(desc: GemmDesc, A_ptr: int, B_ptr: int, C_ptr: int, bias_ptr: int | None = None,
              residual_ptr: int | None = None) -> None:
    """Host-buffer GEMM (``symplex_b200_gemm_host``): copies in, computes, copies out, synchronises."""
    _capi.check(_capi.load().symplex_b200_gemm_host(ctypes.byref(desc), A_ptr, B_ptr, C_ptr, bias_ptr, residual_ptr))


_gemm_descs: dict = {}


def gemm(A, B, *, bias=None, residual=None, activation=None, alpha=1.0, beta=0.0, out=None, out_dtype=None,
         b_layout=ROW_MAJOR, tile_n=0, stream=None, peer_outputs=None):
    """Fused GEMM on CUDA tensors: ``act(alpha * A @ B + beta * residual + bias)``.

    ``A`` is ``[M,K]`` or ``[batch,M,K]``; ``B`` is ``[K,N]`` (``ROW_MAJOR``) or stored as ``[N,K]``
    (``COL_MAJOR``), with the same optional batch dimension. Inputs are both ``torch.float32`` (3xTF32
    path) or both ``torch.bfloat16``. Asynchronous on ``stream`` (default: torch's current stream).

    ``peer_outputs``: device addresses (ints) of up to 7 more buffers with the layout of ``out`` - typically
    the same region of other GPUs' C, mapped into this process - that receive every output tile as well,
    written from inside the kernel (``symplex_b200_gemm_peers``). bf16 inputs only.
    """
    import torch

    if not (A.is_cuda and B.is_cuda):
        raise ValueError("gemm() takes CUDA tensors; use gemm_host()/matmul_jit() for host arrays")
    if A.dtype != B.dtype or A.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"A and B must both be float32 or both bfloat16, got {A.dtype} and {B.dtype}")
    if A.dim() not in (2, 3) or B.dim() != A.dim():
        raise ValueError("A and B must both be 2-D or both 3-D (batched)")
    A = A.contiguous()
    B = B.contiguous()
    batch = A.shape[0] if A.dim() == 3 else 1
    M, K = A.shape[-2], A.shape[-1]
    if b_layout == ROW_MAJOR:
        Kb, N = B.shape[-2], B.shape[-1]
    else:
        N, Kb = B.shape[-2], B.shape[-1]
    if Kb != K or (B.dim() == 3 and B.shape[0] != batch):
        raise ValueError(f"Shape mismatch: A is {tuple(A.shape)}, B is {tuple(B.shape)} (b_layout={b_layout})")
    in_dt = DT_F32 if A.dtype == torch.float32 else DT_BF16
    if out is not None:
        out_t = out.dtype
    else:
        out_t = out_dtype if out_dtype is not None else (torch.float32 if in_dt == DT_F32 else torch.bfloat16)
    if out_t not in (torch.float32, torch.bfloat16):
        raise ValueError("out dtype must be float32 or bfloat16")
    shape = (batch, M, N) if A.dim() == 3 else (M, N)
    if out is None:
        out = torch.empty(shape, device=A.device, dtype=out_t)
    elif tuple(out.shape) != shape or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous tensor of shape {shape}")
    if bias is not None:
        if bias.dtype != torch.float32 or tuple(bias.shape) != (N,):
            raise ValueError(f"bias must be float32 of shape ({N},)")
        bias = bias.contiguous()
    if residual is not None:
        if residual.dtype != out_t or tuple(residual.shape) != shape:
            raise ValueError("residual must match the output's dtype and shape")
        residual = residual.contiguous()
    # Descriptors are only read by the library, so one per distinct problem is built and kept.
    key = (M, N, K, in_dt, out_t, batch, b_layout, alpha, beta, activation, tile_n)
    d = _gemm_descs.get(key)
    if d is None:
        if len(_gemm_descs) >= 512:
            _gemm_descs.clear()
        d = _gemm_descs[key] = make_desc(M, N, K, in_dt, DT_F32 if out_t == torch.float32 else DT_BF16, batch=batch,
                                         b_layout=b_layout, alpha=alpha, beta=beta, activation=activation,
                                         tile_n=tile_n)
    if M == 0 or N == 0 or batch == 0:
        return out
    if K == 0:
        raise ValueError("K == 0 is not supported")
    s = stream if stream is not None else torch.cuda.current_stream(A.device).cuda_stream

    def launch():
        if peer_outputs:
            arr = (ctypes.c_void_p * len(peer_outputs))(*[int(x) for x in peer_outputs])
            return _capi.load().symplex_b200_gemm_peers(ctypes.byref(d), A.data_ptr(), B.data_ptr(), out.data_ptr(),
                                                        bias.data_ptr() if bias is not None else None,
                                                        residual.data_ptr() if residual is not None else None,
                                                        arr, len(peer_outputs), s)
        return _capi.load().symplex_b200_gemm(ctypes.byref(d), A.data_ptr(), B.data_ptr(), out.data_ptr(),
                                              bias.data_ptr() if bias is not None else None,
                                              residual.data_ptr() if residual is not None else None, s)

    # Switching the current device costs several microseconds per call - as much as a small kernel - so it is
    # only done when the operands live on another device than the current one.
    if A.device.index is None or A.device.index == torch.cuda.current_device():
        rc = launch()
    else:
        with torch.cuda.device(A.device):
            rc = launch()
    _capi.check(rc)
    return out


def sync_status(stream=None) -> None:
    """Synchronise and raise if a kernel reported a device-side timeout since the last check."""
    import torch
    s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
    _capi.check(_capi.load().symplex_b200_sync_status(s))


def fused_elementwise(ops, inputs, constants=(), *, reduce_op=_capi.REDUCE_NONE, out=None, stream=None):
    """Run a fused op chain (the reference's ``FusedOpDesc`` program, ``rust-engine/src/x86_emitter.rs:1937-1953``)
    over CUDA ``float32`` (or ``float64``) tensors of equal size and dtype in one kernel.

    ``ops``: ``[(op, lhs_src, lhs_idx, rhs_src, rhs_idx), ...]``. With ``reduce_op`` 255 returns the result
    tensor (``out`` or a new one, shaped like ``inputs[0]``); with 0 / 1 / 2 returns a 0-d ``float64`` CUDA
    tensor holding the sum / max / min. Asynchronous on ``stream`` (default: torch's current stream).
    """
    import torch

    if not inputs:
        raise ValueError("fused_elementwise() needs at least one input tensor")
    n = inputs[0].numel()
    dt = inputs[0].dtype
    if dt not in (torch.float32, torch.float64):
        raise ValueError("inputs must be float32 or float64")
    f64 = dt == torch.float64
    for t in inputs:
        if not t.is_cuda or t.dtype != dt or not t.is_contiguous() or t.numel() != n:
            raise ValueError("inputs must be contiguous CUDA tensors of one dtype and equal size")
    dev = inputs[0].device
    arr = _capi.pack_fused_ops(ops)
    ptrs = (ctypes.c_void_p * len(inputs))(*[t.data_ptr() for t in inputs])
    consts = ((ctypes.c_double if f64 else ctypes.c_float) * max(len(constants), 1))(*[float(c) for c in constants])
    reduce = reduce_op != _capi.REDUCE_NONE
    if reduce:
        res = torch.zeros((), device=dev, dtype=torch.float64)
        dst_ptr, res_ptr = None, res.data_ptr()
    else:
        if out is None:
            out = torch.empty_like(inputs[0])
        elif not out.is_cuda or out.dtype != dt or not out.is_contiguous() or out.numel() != n:
            raise ValueError("out must be a contiguous CUDA tensor of the inputs' dtype and size")
        dst_ptr, res_ptr = out.data_ptr(), None
    s = stream if stream is not None else torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        lib = _capi.load()
        fn = lib.symplex_b200_fused_elementwise_f64 if f64 else lib.symplex_b200_fused_elementwise_f32
        rc = fn(arr, len(ops), ptrs, len(inputs), consts, len(constants), n, int(reduce_op), dst_ptr, res_ptr, s)
    _capi.check(rc)
    return res if reduce else out
