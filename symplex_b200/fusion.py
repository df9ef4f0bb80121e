"""Which op chains fold into the GEMM kernel's epilogue, and what that saves.

Host-side planning only, mirroring the part of the reference's fusion engine that concerns the matmul path
(``rust-engine/src/fusion_engine.rs``): the ``MatMulBiasReLU`` pattern matcher
(``matches_matmul_bias_activation``, :1587-1623), its memory-traffic model (``estimate_memory_savings``,
:1209-1225), its compute-savings constant (:1357) and base confidence (:1885), and the JSON the pyo3
function ``discover_fusions`` returns (``rust-engine/src/lib.rs:344-413``). On top of the reference's
yes/no decision, ``compile_epilogue`` turns a matched chain into the epilogue fields of a
``symplex_gemm_desc`` so the chain really runs as one kernel. The other nine fusion patterns of the
reference are outside this path.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

ACTIVATIONS = ("relu", "gelu", "sigmoid", "tanh", "silu")  # OpType::is_activation, fusion_engine.rs:261-266
MATMULS = ("matmul", "batch_matmul")
DTYPE_BYTES = {"fp32": 4, "fp16": 2, "bf16": 2, "fp8": 1, "int8": 1, "int4": 1}  # DType::size_bytes

COMPUTE_SAVINGS_FACTOR = 1.1   # estimate_compute_savings(MatMulBiasReLU)
BASE_CONFIDENCE = 0.9          # compute_confidence base for MatMulBiasReLU


def matches_matmul_bias_activation(op_types: Sequence[str]) -> bool:
    """``fusion_engine.rs:1587-1623``: [MatMul, Add], [MatMul, act], [MatMul, Add, act], [MatMul, act, *],
    [MatMul, Mul, Add, act]."""
    n = len(op_types)
    if n < 2 or n > 4 or op_types[0] not in MATMULS:
        return False
    if n == 2:
        return op_types[1] == "add" or op_types[1] in ACTIVATIONS
    if n == 3:
        return (op_types[1] == "add" and op_types[2] in ACTIVATIONS) or op_types[1] in ACTIVATIONS
    return op_types[1] == "mul" and op_types[2] == "add" and op_types[3] in ACTIVATIONS


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


def compile_epilogue(op_types: Sequence[str]) -> Optional[Epilogue]:
    """Longest prefix of ``op_types`` (starting at a matmul) that the GEMM kernel executes in its epilogue
    as act(alpha * acc + bias); None if the chain does not start with a matmul."""
    if not op_types or op_types[0] not in MATMULS:
        return None
    i, scale, bias, act = 1, False, False, None
    if i < len(op_types) and op_types[i] == "mul" and i + 1 < len(op_types) and op_types[i + 1] == "add":
        scale, i = True, i + 1
    if i < len(op_types) and op_types[i] == "add":
        bias, i = True, i + 1
    if i < len(op_types) and op_types[i] in ACTIVATIONS:
        act, i = op_types[i], i + 1
    return Epilogue(act, bias, scale, i)


def discover_fusions(ops: Sequence[Tuple[str, Sequence[int], str]]) -> str:
    """JSON with the schema of the reference's ``discover_fusions`` for the matmul-epilogue pattern: every
    maximal chain [matmul, (mul,) (add,) (activation)] of at least two ops becomes one ``MatMulBiasReLU``
    boundary. ``confidence`` is the pattern's base value (the reference adds shape/dtype bonuses)."""
    names = [o[0].lower() for o in ops]
    boundaries: List[dict] = []
    i = 0
    while i < len(ops):
        ep = compile_epilogue(names[i:])
        if ep is not None and ep.consumed >= 2 and matches_matmul_bias_activation(names[i:i + ep.consumed]):
            idx = list(range(i, i + ep.consumed))
            boundaries.append({
                "op_indices": idx,
                "pattern": "MatMulBiasReLU",
                "memory_traffic_savings_bytes": memory_savings_bytes(ops[i:i + ep.consumed]),
                "compute_savings_factor": COMPUTE_SAVINGS_FACTOR,
                "confidence": BASE_CONFIDENCE,
            })
            i += ep.consumed
        else:
            i += 1
    total = sum(b["memory_traffic_savings_bytes"] for b in boundaries)
    return json.dumps({
        "total_hbm_traffic_reduction": total,
        "requires_polyhedral_validation": bool(boundaries),
        "boundaries": boundaries,
    }, indent=2)
