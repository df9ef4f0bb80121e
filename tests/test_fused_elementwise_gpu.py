"""Parity of the fused elementwise kernels (bulk-copy ring kernel and plain-load kernel) with the CPU
oracle's restatement of the reference interpreter (rust-engine/src/x86_emitter.rs:1937-2351), through the
C ABI. Exactly rounded ops (add sub mul div min max neg abs sqrt relu) must match bit for bit; libm-based
ops within a few ulp (rtol 2e-6); sums within 1e-6 relative of the float64 sum; max / min exactly."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ADD, SUB, MUL, DIV, MIN, MAX, NEG, ABS, SQRT, EXP, LOG, SIN, COS, TANH, SIGMOID, RELU = range(16)
IN, CONST, PREV = 0, 1, 2
SUM, RMAX, RMIN, NONE = 0, 1, 2, 255
CHUNK = 2048  # elements per ring stage and input for 3-4 inputs (4096 for 1-2 inputs, 1024 beyond)


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch


def _rng(n, seed=0, lo=-2.0, hi=2.0):
    return np.random.default_rng(seed).uniform(lo, hi, n).astype(np.float32)


def _run(torch, ops, arrays, consts, reduce_op=NONE, misalign=False):
    import symplex_b200 as sx
    dev = []
    for a in arrays:
        if misalign:  # a view that starts 4 bytes past a 16-byte boundary: forces the plain-load kernel
            buf = torch.empty(a.size + 1, device="cuda", dtype=torch.float32)
            t = buf[1:]
            t.copy_(torch.from_numpy(a))
        else:
            t = torch.from_numpy(a).cuda()
        dev.append(t)
    out = sx.fused_elementwise(ops, dev, consts, reduce_op=reduce_op)
    sx.sync_status()
    return out.cpu().numpy() if reduce_op == NONE else float(out.item())


EXACT_PROGRAMS = {
    "axpb": ([(MUL, IN, 0, CONST, 0), (ADD, PREV, 0, CONST, 1)], 1, [2.0, 1.0]),
    "bias_relu": ([(MUL, IN, 0, IN, 1), (ADD, PREV, 0, IN, 2), (RELU, PREV, 1, IN, 0)], 3, []),
    "div_sqrt_abs": ([(ABS, IN, 0, IN, 0), (SQRT, PREV, 0, IN, 0), (ADD, IN, 1, CONST, 0), (ABS, PREV, 2, IN, 0),
                      (DIV, PREV, 1, PREV, 3)], 2, [3.0]),
    "minmax_neg": ([(MIN, IN, 0, IN, 1), (MAX, IN, 0, IN, 1), (NEG, PREV, 0, IN, 0), (SUB, PREV, 1, PREV, 2)], 2, []),
    "slots": ([(MUL, IN, 0, IN, 1), (ADD, IN, 0, IN, 1), (SUB, PREV, 0, PREV, 1), (MUL, PREV, 2, PREV, 0),
               (ADD, PREV, 3, PREV, 1)], 2, []),
    "six_inputs": ([(ADD, IN, 0, IN, 1), (MUL, PREV, 0, IN, 2), (SUB, PREV, 1, IN, 3), (MAX, PREV, 2, IN, 4),
                    (ADD, PREV, 3, IN, 5)], 6, []),
    "no_inputs": ([(ADD, CONST, 0, CONST, 1)], 0, [1.5, 2.25]),
}


@pytest.mark.parametrize("name", sorted(EXACT_PROGRAMS))
@pytest.mark.parametrize("n", [1, 3, CHUNK - 1, CHUNK, CHUNK + 1, 2 * CHUNK - 1, 2 * CHUNK, 2 * CHUNK + 1, 5 * CHUNK + 7,
                               (1 << 20) + 5])
def test_exact_programs_bitwise(torch_cuda, oracle, name, n):
    ops, n_in, consts = EXACT_PROGRAMS[name]
    arrays = [_rng(n, 10 + i) for i in range(max(n_in, 1))]  # at least one array: it fixes n
    want = oracle.fused_elementwise(ops, arrays, consts)
    got = _run(torch_cuda, ops, arrays, consts)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name


@pytest.mark.parametrize("name", ["axpb", "bias_relu", "slots"])
def test_unaligned_arrays_take_the_plain_kernel_bitwise(torch_cuda, oracle, name):
    ops, n_in, consts = EXACT_PROGRAMS[name]
    n = 3 * CHUNK + 11
    arrays = [_rng(n, 20 + i) for i in range(n_in)]
    want = oracle.fused_elementwise(ops, arrays, consts)
    got = _run(torch_cuda, ops, arrays, consts, misalign=True)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("off", [1, 2, 3])
@pytest.mark.parametrize("n", [2, CHUNK + 5, 3 * CHUNK + 11])
def test_equally_misaligned_arrays_take_the_ring_kernel_from_the_next_boundary(torch_cuda, oracle, off, n):
    """Sources and destination all start `off` floats past a 16-byte boundary (x[off:] of aligned arrays): the ring
    kernel runs from the next boundary on and its scalar path computes the 4 - off elements in front of it."""
    import symplex_b200 as sx
    torch = torch_cuda
    ops, n_in, consts = EXACT_PROGRAMS["bias_relu"]
    arrays = [_rng(n, 40 + i) for i in range(n_in)]
    want = oracle.fused_elementwise(ops, arrays, consts)
    dev = []
    for a in arrays:
        t = torch.empty(a.size + off, device="cuda", dtype=torch.float32)[off:]
        t.copy_(torch.from_numpy(a))
        dev.append(t)
    guard = torch.full((n + off + 8,), -7.0, device="cuda", dtype=torch.float32)
    out = guard[off:off + n]
    got = sx.fused_elementwise(ops, dev, consts, out=out)
    sx.sync_status()
    assert got.data_ptr() == out.data_ptr()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert bool((guard[:off] == -7.0).all()) and bool((guard[off + n:] == -7.0).all()), "wrote outside dst"
    # the same arrays reduced: the head elements are part of the sum
    total = float(sx.fused_elementwise(ops, dev, consts, reduce_op=SUM).item())
    assert abs(total - float(want.astype(np.float64).sum())) <= 1e-5 * max(1.0, float(np.abs(want).astype(np.float64).sum()))


def test_libm_ops_within_a_few_ulp(torch_cuda, oracle):
    n = 4 * CHUNK + 3
    x = _rng(n, 30, 0.05, 6.0)
    for op in (EXP, LOG, SIN, COS, TANH, SIGMOID):
        want = oracle.fused_elementwise([(op, IN, 0, IN, 0)], [x], [])
        got = _run(torch_cuda, [(op, IN, 0, IN, 0)], [x], [])
        np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-7, err_msg=f"op {op}")


def test_gelu_tanh_chain(torch_cuda, oracle):
    # 0.5 * x * (1 + tanh(0.79788456 * (x + 0.044715 x^3))) as a 9-op chain with long-lived x.
    ops = [(MUL, IN, 0, IN, 0), (MUL, PREV, 0, IN, 0), (MUL, PREV, 1, CONST, 0), (ADD, PREV, 2, IN, 0),
           (MUL, PREV, 3, CONST, 1), (TANH, PREV, 4, IN, 0), (ADD, PREV, 5, CONST, 2), (MUL, PREV, 6, IN, 0),
           (MUL, PREV, 7, CONST, 3)]
    consts = [0.044715, 0.7978845608, 1.0, 0.5]
    x = _rng(7 * CHUNK + 100, 31, -4, 4)
    want = oracle.fused_elementwise(ops, [x], consts)
    got = _run(torch_cuda, ops, [x], consts)
    np.testing.assert_allclose(got, want, rtol=2e-6, atol=2e-7)


def test_long_program_uses_the_large_parameter_block(torch_cuda, oracle):
    # 200 ops (> 64): x <- x * 1.0001 + 0.001, a hundred times
    ops = []
    for i in range(100):
        ops.append((MUL, IN if i == 0 else PREV, 0 if i == 0 else 2 * i - 1, CONST, 0))
        ops.append((ADD, PREV, 2 * i, CONST, 1))
    x = _rng(2 * CHUNK + 5, 32)
    want = oracle.fused_elementwise(ops, [x], [1.0001, 0.001])
    got = _run(torch_cuda, ops, [x], [1.0001, 0.001])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("n", [5, 64, CHUNK, 4 * CHUNK + 64, 4 * CHUNK + 67, (1 << 21) + 13])
@pytest.mark.parametrize("misalign", [False, True])
def test_reductions(torch_cuda, oracle, n, misalign):
    x, y = _rng(n, 40), _rng(n, 41)
    ops = [(MUL, IN, 0, IN, 1), (ADD, PREV, 0, CONST, 0)]
    vals = (x * y + np.float32(0.25)).astype(np.float64)
    got = _run(torch_cuda, ops, [x, y], [0.25], reduce_op=SUM, misalign=misalign)
    assert abs(got - vals.sum()) <= 1e-6 * np.abs(vals).sum()
    ref = oracle.fused_elementwise(ops, [x, y], [0.25], reduce_op=SUM)
    assert abs(got - ref) <= 2e-5 * np.abs(vals).sum()  # the reference's 32 fp32 lanes are the less accurate side
    for rop in (RMAX, RMIN):
        got = _run(torch_cuda, ops, [x, y], [0.25], reduce_op=rop, misalign=misalign)
        assert got == oracle.fused_elementwise(ops, [x, y], [0.25], reduce_op=rop, exact=True)
        if n % 8 == 0:  # no scalar tail: the reference's own value is the true extremum too
            assert got == oracle.fused_elementwise(ops, [x, y], [0.25], reduce_op=rop)


def test_sum_is_reproducible_and_counts_every_element(torch_cuda):
    import symplex_b200 as sx
    torch = torch_cuda
    n = (1 << 26) + 12345  # 268 MB per array: several sweeps of the persistent grid
    x = torch.rand(n, device="cuda", dtype=torch.float32)
    ones = sx.fused_elementwise([(MUL, IN, 0, CONST, 0), (ADD, PREV, 0, CONST, 1)], [x], [0.0, 1.0], reduce_op=SUM)
    assert float(ones.item()) == float(n)
    a = sx.fused_elementwise([(MUL, IN, 0, IN, 0)], [x], [], reduce_op=SUM).item()
    b = sx.fused_elementwise([(MUL, IN, 0, IN, 0)], [x], [], reduce_op=SUM).item()
    assert a == b
    want = float((x.double() ** 2).sum().item())
    assert abs(a - want) <= 1e-6 * want
    sx.sync_status()


def test_output_may_alias_an_input(torch_cuda, oracle):
    import symplex_b200 as sx
    torch = torch_cuda
    x = _rng(3 * CHUNK + 9, 50)
    t = torch.from_numpy(x).cuda()
    sx.fused_elementwise([(MUL, IN, 0, CONST, 0), (ADD, PREV, 0, CONST, 1)], [t], [2.0, 1.0], out=t)
    sx.sync_status()
    want = oracle.fused_elementwise([(MUL, IN, 0, CONST, 0), (ADD, PREV, 0, CONST, 1)], [x], [2.0, 1.0])
    assert np.array_equal(t.cpu().numpy(), want)


def test_host_entry_points(torch_cuda, oracle):
    from symplex_b200 import _symplex_core, engine
    n = (9 << 20) + 77  # two pipeline chunks plus a ragged end
    a, b = _rng(n, 60), _rng(n, 61, 0.5, 2.0)
    ops = [(DIV, IN, 0, IN, 1), (SUB, PREV, 0, CONST, 0)]
    dst = np.empty(n, np.float32)
    r = _symplex_core.simd_fused_elementwise_f32(ops, [a.ctypes.data, b.ctypes.data], [0.5], n, NONE, dst.ctypes.data)
    assert r == 0.0
    assert np.array_equal(dst, oracle.fused_elementwise(ops, [a, b], [0.5]))
    s = _symplex_core.simd_fused_elementwise_f32(ops, [a.ctypes.data, b.ctypes.data], [0.5], n, SUM, 0)
    want = (a / b - np.float32(0.5)).astype(np.float64)
    assert abs(s - want.sum()) <= 1e-6 * np.abs(want).sum()
    m = _symplex_core.simd_fused_elementwise_f32(ops, [a.ctypes.data, b.ctypes.data], [0.5], n, RMAX, 0)
    assert m == float(want.max())
    out = np.empty(n, np.float32)
    for name, fn in [("add", np.add), ("sub", np.subtract), ("mul", np.multiply), ("div", np.divide),
                     ("min", np.minimum), ("max", np.maximum)]:
        assert engine.cuda_elementwise_raw(a.ctypes.data, b.ctypes.data, out.ctypes.data, n, name) == 0
        assert np.array_equal(out, fn(a, b)), name


# ----------------------------------------------------------------------------- the f64 twin

def _run64(torch, ops, arrays, consts, reduce_op=NONE, misalign=False):
    import symplex_b200 as sx
    dev = []
    for a in arrays:
        if misalign:  # 8 bytes past a 16-byte boundary
            buf = torch.empty(a.size + 1, device="cuda", dtype=torch.float64)
            t = buf[1:]
            t.copy_(torch.from_numpy(a))
        else:
            t = torch.from_numpy(a).cuda()
        dev.append(t)
    out = sx.fused_elementwise(ops, dev, consts, reduce_op=reduce_op)
    sx.sync_status()
    return out.cpu().numpy() if reduce_op == NONE else float(out.item())


@pytest.mark.parametrize("name", ["axpb", "bias_relu", "div_sqrt_abs", "slots", "six_inputs"])
@pytest.mark.parametrize("n", [1, 1023, 1024, 1025, 2048, 5 * 2048 + 7, (1 << 19) + 3])
def test_f64_exact_programs_bitwise(torch_cuda, oracle, name, n):
    ops, n_in, consts = EXACT_PROGRAMS[name]
    arrays = [np.random.default_rng(70 + i).uniform(-2, 2, n) for i in range(n_in)]
    want = oracle.fused_elementwise(ops, arrays, consts, dtype=np.float64)
    for misalign in (False, True):
        got = _run64(torch_cuda, ops, arrays, consts, misalign=misalign)
        assert got.dtype == np.float64 and np.array_equal(got.view(np.uint64), want.view(np.uint64)), (name, misalign)


def test_f64_libm_ops_and_reductions(torch_cuda, oracle):
    n = 3 * 2048 + 5
    x = np.random.default_rng(80).uniform(0.05, 6.0, n)
    for op in (EXP, LOG, SIN, COS, TANH, SIGMOID):
        want = oracle.fused_elementwise([(op, IN, 0, IN, 0)], [x], [], dtype=np.float64)
        got = _run64(torch_cuda, [(op, IN, 0, IN, 0)], [x], [])
        np.testing.assert_allclose(got, want, rtol=1e-14, atol=1e-15, err_msg=f"op {op}")
    y = np.random.default_rng(81).uniform(-2, 2, n)
    ops = [(MUL, IN, 0, IN, 1), (ADD, PREV, 0, CONST, 0)]
    vals = x * y + 0.25
    got = _run64(torch_cuda, ops, [x, y], [0.25], reduce_op=SUM)
    assert abs(got - np.sum(vals)) <= 1e-13 * np.abs(vals).sum()
    assert abs(got - oracle.fused_elementwise(ops, [x, y], [0.25], reduce_op=SUM, dtype=np.float64)) <= 1e-12 * np.abs(vals).sum()
    assert _run64(torch_cuda, ops, [x, y], [0.25], reduce_op=RMAX) == vals.max()
    assert _run64(torch_cuda, ops, [x, y], [0.25], reduce_op=RMIN, misalign=True) == vals.min()


def test_f64_host_entry_point(torch_cuda, oracle):
    from symplex_b200 import _symplex_core
    n = (5 << 20) + 3  # two pipeline chunks (4 Mi doubles each) plus a ragged end
    a = np.random.default_rng(90).uniform(-2, 2, n)
    b = np.random.default_rng(91).uniform(0.5, 2, n)
    ops = [(DIV, IN, 0, IN, 1), (SUB, PREV, 0, CONST, 0)]
    dst = np.empty(n, np.float64)
    assert _symplex_core.simd_fused_elementwise_f64(ops, [a.ctypes.data, b.ctypes.data], [0.5], n, NONE, dst.ctypes.data) == 0.0
    assert np.array_equal(dst, a / b - 0.5)
    s = _symplex_core.simd_fused_elementwise_f64(ops, [a.ctypes.data, b.ctypes.data], [0.5], n, SUM, 0)
    assert abs(s - np.sum(dst)) <= 1e-13 * np.abs(dst).sum()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_random_programs_bitwise(torch_cuda, oracle, dtype):
    """Seeded random chains over the exactly rounded, overflow-safe ops (add sub mul min max neg abs relu), random
    operand sources including long-lived intermediates, 1-6 inputs, ragged lengths: bit for bit against the oracle."""
    import symplex_b200 as sx
    torch = torch_cuda
    rng = np.random.default_rng(77)
    safe = [ADD, SUB, MUL, MIN, MAX, NEG, ABS, RELU]
    for trial in range(40):
        n_inputs = int(rng.integers(1, 7))
        n_ops = int(rng.integers(1, 14))
        n = int(rng.choice([37, 1000, 4096, 5000, 12289, 40000]))
        consts = [float(c) for c in rng.uniform(-1.5, 1.5, 3)]
        ops = []
        for i in range(n_ops):
            def operand():
                src = int(rng.choice([0, 0, 1, 2, 2]))
                if src == 0:
                    return 0, int(rng.integers(0, n_inputs))
                if src == 1:
                    return 1, int(rng.integers(0, 3))
                return (2, int(rng.integers(0, i))) if i > 0 else (0, 0)
            (ls, li), (rs, ri) = operand(), operand()
            ops.append((int(rng.choice(safe)), ls, li, rs, ri))
        arrays = [rng.uniform(-1.2, 1.2, n).astype(dtype) for _ in range(n_inputs)]
        want = oracle.fused_elementwise(ops, arrays, consts, dtype=dtype)
        got = sx.fused_elementwise(ops, [torch.from_numpy(a).cuda() for a in arrays], consts).cpu().numpy()
        bits = np.uint32 if dtype == np.float32 else np.uint64
        assert np.array_equal(got.view(bits), want.view(bits)), (trial, ops)
        ref_sum = oracle.fused_elementwise(ops, arrays, consts, reduce_op=SUM, dtype=dtype)
        got_sum = float(sx.fused_elementwise(ops, [torch.from_numpy(a).cuda() for a in arrays], consts,
                                             reduce_op=SUM).item())
        scale = float(np.abs(want.astype(np.float64)).sum()) + 1e-30
        assert abs(got_sum - float(want.astype(np.float64).sum())) <= (1e-6 if dtype == np.float32 else 1e-13) * scale
        assert abs(got_sum - ref_sum) <= 2e-5 * scale
    sx.sync_status()
