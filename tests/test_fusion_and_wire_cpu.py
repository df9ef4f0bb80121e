"""Host logic next to the GEMM path: the matmul-epilogue fusion matcher (against the reference's own unit-test
vectors) and decoding of the TensorMatMul wire record (error paths only - no GPU here)."""
import ctypes
import json
import struct

import pytest

from symplex_b200 import _capi, fusion


def test_reference_kat_matmul_bias_relu_boundary():
    # rust-engine/src/fusion_engine.rs:2469-2483
    ops = [("matmul", [128, 256], "fp16"), ("add", [128, 256], "fp16"), ("relu", [128, 256], "fp16")]
    d = json.loads(fusion.discover_fusions(ops))
    assert len(d["boundaries"]) == 1
    b = d["boundaries"][0]
    assert b["pattern"] == "MatMulBiasReLU" and b["op_indices"] == [0, 1, 2]
    assert d["total_hbm_traffic_reduction"] > 0 and d["requires_polyhedral_validation"] is True


def test_reference_kat_memory_savings():
    # rust-engine/src/fusion_engine.rs:2558-2573: 2*65536 + 2*65536
    ops = [("matmul", [128, 256], "fp16"), ("add", [128, 256], "fp16"), ("relu", [128, 256], "fp16")]
    assert fusion.memory_savings_bytes(ops) == 2 * 65536 + 2 * 65536 == 262144


@pytest.mark.parametrize("chain,ok", [
    (["matmul", "add"], True), (["matmul", "gelu"], True), (["matmul", "add", "relu"], True),
    (["batch_matmul", "add", "silu"], True), (["matmul", "mul", "add", "tanh"], True),
    (["matmul", "relu", "add"], True),          # [MatMul, activation, *]
    (["matmul"], False), (["add", "relu"], False), (["matmul", "mul", "relu"], False),
    (["matmul", "add", "add"], False), (["matmul", "mul", "add", "add"], False),
    (["matmul", "add", "relu", "mul", "add"], False),
])
def test_pattern_matcher(chain, ok):
    assert fusion.matches_matmul_bias_activation(chain) is ok


def test_compile_epilogue():
    ep = fusion.compile_epilogue(["matmul", "mul", "add", "gelu", "softmax"])
    assert (ep.activation, ep.has_bias, ep.has_scale, ep.consumed) == ("gelu", True, True, 4)
    ep = fusion.compile_epilogue(["matmul", "sigmoid"])
    assert (ep.activation, ep.has_bias, ep.has_scale, ep.consumed) == ("sigmoid", False, False, 2)
    assert fusion.compile_epilogue(["add", "relu"]) is None
    d = json.loads(fusion.discover_fusions([("matmul", [8, 8], "bf16"), ("softmax", [8, 8], "bf16"),
                                            ("matmul", [8, 8], "bf16"), ("add", [8, 8], "bf16")]))
    assert [b["op_indices"] for b in d["boundaries"]] == [[2, 3]]


def _record(dst, lhs, rhs, m, n, k, ety, ll, rl, opcode=0xA2):
    return struct.pack("<BHHHQQQBBB", opcode, dst, lhs, rhs, m, n, k, ety, ll, rl)


def test_tensor_matmul_record_layout_and_errors(lib):
    rec = _record(2, 0, 1, 4, 4, 4, 9, 0, 0)
    assert len(rec) == 34  # rust-engine/src/types.rs:884-904
    slots = (ctypes.c_void_p * 3)()
    f = lib.symplex_b200_exec_tensor_matmul
    assert f(rec[:20], 20, slots, 3) == _capi.ERR_INVALID
    assert f(_record(2, 0, 1, 4, 4, 4, 9, 0, 0, opcode=0x70), 34, slots, 3) == _capi.ERR_INVALID
    assert f(_record(5, 0, 1, 4, 4, 4, 9, 0, 0), 34, slots, 3) == _capi.ERR_INVALID   # slot out of range
    assert f(_record(2, 0, 1, 4, 4, 4, 12, 0, 0), 34, slots, 3) == _capi.ERR_INVALID  # element type not on this path
    assert f(_record(2, 0, 1, 4, 4, 4, 10, 0, 1), 34, slots, 3) == _capi.ERR_INVALID  # F64 takes a row-major rhs
    assert f(_record(2, 0, 1, 4, 4, 4, 10, 0, 0), 34, slots, 3) == _capi.ERR_INVALID  # F64: null slot pointers
    assert f(_record(2, 0, 1, 4, 4, 4, 9, 1, 0), 34, slots, 3) == _capi.ERR_INVALID   # col-major lhs
    assert f(_record(2, 0, 1, 4, 4, 4, 9, 0, 7), 34, slots, 3) == _capi.ERR_INVALID
    assert f(_record(2, 0, 1, 0, 4, 4, 9, 0, 0), 34, slots, 3) == 0                   # zero dimension: no-op
