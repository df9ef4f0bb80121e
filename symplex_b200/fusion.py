"""Which op chains fold into the GEMM kernel's epilogue, and what that saves.

Host-side planning only, mirroring the part of the reference's fusion engine that concerns the matmul path
(``rust-engine/src/fusion_engine.rs``): the ``MatMulBiasReLU`` pattern matcher
(``matches_matmul_bias_activation``, :1587-1623), its memory-traffic model (``estimate_memory_savings``,
:1209-1225), its compute-savings constant (:1357), confidence rule (:1882-1965) and the JSON the pyo3 function
``discover_fusions`` returns (``rust-engine/src/lib.rs:344-413``). The decisions are made by the library
(``symplex_b200_discover_fusions`` / ``symplex_b200_compile_epilogue``, C ABI, no GPU needed); this module is the
Python face of those two functions, as the reference's pyo3 function is of its Rust engine. ``compile_epilogue``
turns a matched chain into the epilogue fields of a ``symplex_gemm_desc`` so the chain really runs as one
kernel. The other nine fusion patterns of the reference are outside this path.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

from . import _capi

ACTIVATIONS = ("relu", "gelu", "sigmoid", "tanh", "silu")  # OpType::is_activation, fusion_engine.rs:261-266
MATMULS = ("matmul", "batch_matmul")
DTYPE_BYTES = {"fp32": 4, "fp16": 2, "bf16": 2, "fp8": 1, "int8": 1, "int4": 1}  # DType::size_bytes
_ACT_NAMES = {v: k for k, v in _capi.ACTIVATIONS.items() if isinstance(k, str) and k != "none"}


def _as_ops(op_types: Sequence[str]):
    return [(t, [1], "fp32") for t in op_types]


def matches_matmul_bias_activation(op_types: Sequence[str]) -> bool:
    """``fusion_engine.rs:1587-1623``: [MatMul, Add], [MatMul, act], [MatMul, Add, act], [MatMul, act, *],
    [MatMul, Mul, Add, act]. Pure predicate on the names (the same rule the library applies to the chains it
    extracts)."""
    t = [x.lower() for x in op_types]
    n = len(t)
    if n < 2 or n > 4 or t[0] not in MATMULS:
        return False
    if n == 2:
        return t[1] == "add" or t[1] in ACTIVATIONS
    if n == 3:
        return (t[1] == "add" and t[2] in ACTIVATIONS) or t[1] in ACTIVATIONS
    return t[1] == "mul" and t[2] == "add" and t[3] in ACTIVATIONS


def memory_savings_bytes(ops: Sequence[Tuple[str, Sequence[int], str]]) -> int:
    """``fusion_engine.rs:1209-1225``: the MatMul output and the Add output each cost one write and one read
    when the chain is not fused: 2 * bytes(op 0) + 2 * bytes(op 1)."""
    def nbytes(op):
        _, shape, dtype = op
        total = 1
        for d in shape:
            total *= int(d)
        return total * DTYPE_BYTES.get(dtype.lower(), 4)
    first = nbytes(ops[0]) if ops else 0
    second = nbytes(ops[1]) if len(ops) >= 2 else 0
    return 2 * first + 2 * second


@dataclass
class Epilogue:
    """Epilogue fields of a ``symplex_gemm_desc`` for a fused chain, and how many ops it consumed."""
    activation: Optional[str]
    has_bias: bool
    has_scale: bool
    consumed: int


def compile_epilogue(op_types: Sequence[str], desc: Optional[_capi.GemmDesc] = None) -> Optional[Epilogue]:
    """Longest prefix of ``op_types`` (starting at a matmul) that the GEMM kernel executes in its epilogue
    as act(alpha * acc + bias); None if the chain does not start with a matmul. With ``desc`` given, its
    ``activation`` field is set (``symplex_b200_compile_epilogue``)."""
    if not op_types:
        return None
    arr, _keep = _capi.pack_fusion_ops(_as_ops(op_types))
    d = desc if desc is not None else _capi.GemmDesc()
    consumed, bias, scale = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    rc = _capi.load().symplex_b200_compile_epilogue(arr, len(op_types), 0, ctypes.byref(d), ctypes.byref(consumed),
                                                    ctypes.byref(bias), ctypes.byref(scale))
    if rc != 0:
        return None
    return Epilogue(_ACT_NAMES.get(d.activation), bool(bias.value), bool(scale.value), consumed.value)


def discover_fusions(ops: Sequence[Tuple[str, Sequence[int], str]]) -> str:
    """JSON with the schema of the reference's ``discover_fusions`` for the matmul-epilogue pattern: every
    maximal chain [matmul, (mul,) (add,) (activation)] of at least two ops becomes one ``MatMulBiasReLU``
    boundary (``symplex_b200_discover_fusions``)."""
    ops = list(ops)
    arr, _keep = _capi.pack_fusion_ops(ops)
    lib = _capi.load()
    cap = 1024 + 256 * len(ops)
    buf = ctypes.create_string_buffer(cap)
    n = lib.symplex_b200_discover_fusions(arr, len(ops), buf, cap)
    if n < 0:
        raise _capi.SymplexB200Error(int(n), _capi.last_error())
    return buf.value.decode()
