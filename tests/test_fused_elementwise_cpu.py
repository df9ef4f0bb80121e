"""Fused elementwise chains, CPU side: the oracle's restatement of the reference interpreter
(rust-engine/src/x86_emitter.rs:1937-2351) against NumPy, and the library's host-side program compiler
(slot assignment, limits, error codes). No GPU compute here."""
import ctypes

import numpy as np
import pytest

from symplex_b200 import _capi, engine

ADD, SUB, MUL, DIV, MIN, MAX, NEG, ABS, SQRT, EXP, LOG, SIN, COS, TANH, SIGMOID, RELU = range(16)
IN, CONST, PREV = 0, 1, 2
SUM, RMAX, RMIN, NONE = 0, 1, 2, 255


def _rng(n, seed=0, lo=-2.0, hi=2.0):
    return np.random.default_rng(seed).uniform(lo, hi, n).astype(np.float32)


# ----------------------------------------------------------------------------- oracle vs NumPy

def test_axpb_matches_numpy_bitwise(oracle):
    # The reference's documented example chain: x * 2.0 + 1.0 (x86_emitter.rs:1929-1931).
    x = _rng(1000)
    got = oracle.fused_elementwise([(MUL, IN, 0, CONST, 0), (ADD, PREV, 0, CONST, 1)], [x], [2.0, 1.0])
    want = (x * np.float32(2.0)) + np.float32(1.0)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("n", [1, 7, 8, 31, 32, 33, 77, 1000])
def test_binary_ops_bitwise(oracle, n):
    a, b = _rng(n, 1), _rng(n, 2, 0.5, 3.0)
    for op, fn in [(ADD, np.add), (SUB, np.subtract), (MUL, np.multiply), (DIV, np.divide), (MIN, np.minimum),
                   (MAX, np.maximum)]:
        got = oracle.fused_elementwise([(op, IN, 0, IN, 1)], [a, b], [])
        assert np.array_equal(got, fn(a, b)), op


def test_unary_ops(oracle):
    x = _rng(513, 3, 0.1, 4.0)
    exact = {NEG: -x, ABS: np.abs(x), SQRT: np.sqrt(x), RELU: np.maximum(x - 2, 0)}
    assert np.array_equal(oracle.fused_elementwise([(NEG, IN, 0, IN, 0)], [x], []), exact[NEG])
    assert np.array_equal(oracle.fused_elementwise([(ABS, IN, 0, IN, 0)], [-x], []), exact[ABS])
    assert np.array_equal(oracle.fused_elementwise([(SQRT, IN, 0, IN, 0)], [x], []), exact[SQRT])
    assert np.array_equal(oracle.fused_elementwise([(SUB, IN, 0, CONST, 0), (RELU, PREV, 0, IN, 0)], [x], [2.0]),
                          exact[RELU])
    x64 = x.astype(np.float64)
    for op, fn in [(EXP, np.exp), (LOG, np.log), (SIN, np.sin), (COS, np.cos), (TANH, np.tanh),
                   (SIGMOID, lambda v: 1 / (1 + np.exp(-v)))]:
        got = oracle.fused_elementwise([(op, IN, 0, IN, 0)], [x], [])
        np.testing.assert_allclose(got, fn(x64), rtol=3e-7, atol=1e-7, err_msg=str(op))


def test_unknown_opcode_passes_lhs_and_bad_indices_read_zero(oracle):
    x = _rng(40, 4)
    assert np.array_equal(oracle.fused_elementwise([(99, IN, 0, IN, 0)], [x], []), x)
    # input 5 and constant 9 do not exist: both read as 0.0
    got = oracle.fused_elementwise([(ADD, IN, 5, CONST, 9), (ADD, PREV, 0, IN, 0)], [x], [1.0])
    assert np.array_equal(got, x)
    # op 0 refers to op 1 (not computed yet): reads 0.0
    got = oracle.fused_elementwise([(ADD, IN, 0, PREV, 1), (MUL, PREV, 0, CONST, 0)], [x], [3.0])
    assert np.array_equal(got, x * np.float32(3.0))


def test_sum_lane_structure_exact_on_integers(oracle):
    # Integers below 2^24 add exactly in fp32 in any order: the lane structure must still visit every element once.
    for n in [1, 5, 8, 33, 77, 1000, 4099]:
        x = np.arange(1, n + 1, dtype=np.float32)
        got = oracle.fused_elementwise([(MUL, IN, 0, CONST, 0)], [x], [2.0], reduce_op=SUM)
        assert got == float(n * (n + 1)), n


def test_sum_against_float64(oracle):
    x = _rng(100003, 5)
    got = oracle.fused_elementwise([(MUL, IN, 0, IN, 0)], [x], [], reduce_op=SUM)
    assert abs(got - float(np.sum(x.astype(np.float64) ** 2))) < 1e-5 * got


def test_max_min_without_tail_and_the_reference_tail_quirk(oracle):
    x = _rng(64, 6)
    assert oracle.fused_elementwise([(ADD, IN, 0, CONST, 0)], [x], [0.0], reduce_op=RMAX) == float(x.max())
    assert oracle.fused_elementwise([(ADD, IN, 0, CONST, 0)], [x], [0.0], reduce_op=RMIN) == float(x.min())
    # n % 8 != 0: the reference returns (max of the vector part) + (max of the scalar tail), x86_emitter.rs:2347.
    y = _rng(67, 7)
    ref_value = oracle.fused_elementwise([(ADD, IN, 0, CONST, 0)], [y], [0.0], reduce_op=RMAX)
    assert ref_value == float(y[:64].max()) + float(y[64:].max())
    assert oracle.fused_elementwise([(ADD, IN, 0, CONST, 0)], [y], [0.0], reduce_op=RMAX, exact=True) == float(y.max())
    assert oracle.fused_elementwise([(ADD, IN, 0, CONST, 0)], [y], [0.0], reduce_op=RMIN, exact=True) == float(y.min())
    z = _rng(5, 8)
    assert oracle.fused_elementwise([(ADD, IN, 0, CONST, 0)], [z], [0.0], reduce_op=RMIN, exact=True) == float(z.min())


# ----------------------------------------------------------------------------- host-side program compiler

def _info(lib, ops, n_inputs):
    arr = _capi.pack_fused_ops(ops)
    slots, used = ctypes.c_int(-1), ctypes.c_int(-1)
    rc = lib.symplex_b200_fused_program_info(arr, len(ops), n_inputs, ctypes.byref(slots), ctypes.byref(used))
    return rc, slots.value, used.value


def test_fused_op_struct_is_the_reference_layout():
    assert ctypes.sizeof(_capi.FusedOp) == 8
    assert _capi.FusedOp.lhs_idx.offset == 2 and _capi.FusedOp.rhs_src.offset == 4 and _capi.FusedOp.rhs_idx.offset == 6


def test_chain_needs_no_slots(lib):
    # every value is consumed by the next op: all stay in registers
    ops = [(MUL, IN, 0, CONST, 0), (ADD, PREV, 0, CONST, 1), (RELU, PREV, 1, IN, 0)]
    assert _info(lib, ops, 1) == (0, 0, 1)


def test_slots_are_assigned_by_liveness_and_reused(lib):
    # t0 = a*b ; t1 = a+b ; t2 = t0-t1 ; t3 = t2*t0   -> only t0 outlives its successor
    ops = [(MUL, IN, 0, IN, 1), (ADD, IN, 0, IN, 1), (SUB, PREV, 0, PREV, 1), (MUL, PREV, 2, PREV, 0)]
    assert _info(lib, ops, 2) == (0, 1, 2)
    # 40 values each used two ops later: two slots suffice
    ops = [(ADD, IN, 0, CONST, 0), (ADD, IN, 0, CONST, 0)]
    for i in range(2, 42):
        ops.append((ADD, PREV, i - 2, PREV, i - 1))
    rc, slots, used = _info(lib, ops, 1)
    assert rc == 0 and slots <= 2 and used == 1


def test_unused_inputs_are_not_counted(lib):
    assert _info(lib, [(ADD, IN, 3, IN, 7)], 9) == (0, 0, 2)
    assert _info(lib, [(ADD, IN, 3, IN, 3)], 9) == (0, 0, 1)
    assert _info(lib, [(NEG, IN, 0, IN, 5)], 9) == (0, 0, 1)  # unary: rhs ignored


def test_limits_are_reported(lib):
    assert _info(lib, [], 1)[0] == _capi.ERR_INVALID
    too_long = [(ADD, IN, 0, CONST, 0)] * 1025
    assert _info(lib, too_long, 1)[0] == _capi.ERR_INVALID
    assert "1024" in _capi.last_error()
    assert _info(lib, [(ADD, IN, 0, CONST, 0)] * 1024, 1)[0] == 0
    many_inputs = [(ADD, IN, 0, IN, 1)] + [(ADD, PREV, i - 1, IN, i + 1) for i in range(1, 17)]
    assert _info(lib, many_inputs, 32)[0] == _capi.ERR_INVALID
    assert "16 distinct input" in _capi.last_error()
    # 18 values all consumed at the very end: more than 16 alive at once
    ops = [(ADD, IN, 0, CONST, 0) for _ in range(18)]
    ops += [(ADD, PREV, 0, PREV, 1)] + [(ADD, PREV, 17 + i, PREV, i + 1) for i in range(1, 17)]
    assert _info(lib, ops, 1)[0] == _capi.ERR_INVALID
    assert "alive" in _capi.last_error()


def test_elementwise_raw_argument_handling(lib):
    a = np.zeros(4, np.float32)
    assert engine.cuda_elementwise_raw(a.ctypes.data, a.ctypes.data, a.ctypes.data, 0, "add") == 0
    assert engine.cuda_elementwise_raw(a.ctypes.data, a.ctypes.data, a.ctypes.data, 4, "pow") == -2
    if not lib.symplex_cuda_available():  # no CPU fallback: a real request fails without a B200
        assert engine.cuda_elementwise_raw(a.ctypes.data, a.ctypes.data, a.ctypes.data, 4, "add") == -1


def test_empty_requests_return_zero_without_a_gpu(lib):
    from symplex_b200 import _symplex_core
    assert _symplex_core.simd_fused_elementwise_f32([], [], [], 10, SUM, 0) == 0.0
    assert _symplex_core.simd_fused_elementwise_f32([(ADD, IN, 0, IN, 0)], [0], [], 0, SUM, 0) == 0.0


# ----------------------------------------------------------------------------- the f64 twin

def test_f64_chain_matches_numpy_bitwise(oracle):
    x = np.random.default_rng(9).uniform(-2, 2, 1003)
    y = np.random.default_rng(10).uniform(0.5, 2, 1003)
    got = oracle.fused_elementwise([(MUL, IN, 0, CONST, 0), (ADD, PREV, 0, CONST, 1), (DIV, PREV, 1, IN, 1)], [x, y],
                                   [2.0, 1.0], dtype=np.float64)
    assert got.dtype == np.float64 and np.array_equal(got, (x * 2.0 + 1.0) / y)
    got = oracle.fused_elementwise([(SQRT, IN, 0, IN, 0), (NEG, PREV, 0, IN, 0)], [y], [], dtype=np.float64)
    assert np.array_equal(got, -np.sqrt(y))


def test_f64_reduction_lane_structure(oracle):
    for n in [1, 3, 4, 15, 16, 17, 100, 1003]:
        x = np.arange(1, n + 1, dtype=np.float64)
        assert oracle.fused_elementwise([(MUL, IN, 0, CONST, 0)], [x], [2.0], reduce_op=SUM, dtype=np.float64) == n * (n + 1)
    y = np.random.default_rng(11).uniform(-2, 2, 64)
    assert oracle.fused_elementwise([(ADD, IN, 0, CONST, 0)], [y], [0.0], reduce_op=RMAX, dtype=np.float64) == y.max()
    z = np.random.default_rng(12).uniform(-2, 2, 67)  # tail of 3: the reference adds the two partial maxima
    assert oracle.fused_elementwise([(ADD, IN, 0, CONST, 0)], [z], [0.0], reduce_op=RMAX, dtype=np.float64) == \
        z[:64].max() + z[64:].max()
    assert oracle.fused_elementwise([(ADD, IN, 0, CONST, 0)], [z], [0.0], reduce_op=RMIN, exact=True,
                                    dtype=np.float64) == z.min()


def _expected_slots_and_inputs(ops, n_inputs):
    """Independent restatement of the host compiler's bookkeeping: a value needs a slot iff it is used by an op
    other than its immediate successor; a slot is released at the value's last use, before the using op's own
    result is placed; slots are taken lowest-free-first is not required - only the high-water mark is compared."""
    n = len(ops)
    refs = []
    used_inputs = set()
    for i, (op, ls, li, rs, ri) in enumerate(ops):
        r = []
        sides = [(ls, li)] if op >= 6 else [(ls, li), (rs, ri)]
        for src, idx in sides:
            if src == 0 and idx < n_inputs:
                used_inputs.add(idx)
            elif src == 2 and idx < i:
                r.append(idx)
        refs.append(r)
    last_use = [-1] * n
    for i, r in enumerate(refs):
        for j in r:
            last_use[j] = i
    live, high = set(), 0
    for i in range(n):
        for j in set(refs[i]):
            if last_use[j] == i:
                live.discard(j)
        if last_use[i] > i + 1:
            live.add(i)
            high = max(high, len(live))
    return high, len(used_inputs)


def test_program_compiler_against_an_independent_liveness_count(lib):
    rng = np.random.default_rng(123)
    checked = 0
    for trial in range(300):
        n_ops = int(rng.integers(1, 40))
        n_inputs = int(rng.integers(1, 6))
        ops = []
        for i in range(n_ops):
            op = int(rng.integers(0, 17))
            def operand():
                src = int(rng.choice([0, 1, 2, 2]))
                if src == 0:
                    return 0, int(rng.integers(0, n_inputs + 1))          # sometimes out of range: reads 0
                if src == 1:
                    return 1, int(rng.integers(0, 3))
                return 2, int(rng.integers(0, max(1, i + 1)))             # sometimes a self / forward reference
            (ls, li), (rs, ri) = operand(), operand()
            ops.append((op, ls, li, rs, ri))
        want_slots, want_inputs = _expected_slots_and_inputs(ops, n_inputs)
        rc, slots, used = _info(lib, ops, n_inputs)
        if want_slots > 16:
            assert rc == _capi.ERR_INVALID
            continue
        assert (rc, slots, used) == (0, want_slots, want_inputs), (trial, ops)
        checked += 1
    assert checked > 250
