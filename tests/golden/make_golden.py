"""Regenerate tests/golden/*.npz from the reference itself (run where the reference checkout exists).

    python tests/golden/make_golden.py /path/to/reference

Two sources, both the reference's own code, neither modified:
  * its Python package imported in pure-Python mode (python/symplex): ``matmul_jit`` / ``matmul_tiled`` /
    ``matmul`` and the DeviceArray activations ``gelu`` / ``relu`` / ``sigmoid`` / ``tanh``;
  * its C kernel library kernels/matmul.c compiled unchanged (oracle/_ref/libsymplex_kernels.so, built by
    oracle/Makefile): ``symplex_matmul_f32`` and ``symplex_matmul_tiled_f32``.
  * fused elementwise chains (the programs the reference's interpreter simd_fused_elementwise_f32 / _f64 runs,
    rust-engine/src/x86_emitter.rs:1937-2470) evaluated by the reference's own Python layer: ``@symplex.jit``
    functions which, without the native core, execute their trace op by op through NumPy
    (python/symplex/_jit.py:1329-1330, 1740-1760) - the same separately rounded IEEE operations per element.
Inputs are seeded; every array needed to replay a case is stored next to the reference's output.
"""
import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if len(sys.argv) < 2:
    sys.exit(__doc__)
REF = sys.argv[1]


def main():
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(REF, "python"))
    import symplex  # the reference package, pure-Python fallback mode

    ref_so = os.path.join(ROOT, "oracle", "_ref", "libsymplex_kernels.so")
    ref_c = ctypes.CDLL(ref_so)
    i64 = ctypes.c_int64

    def c_matmul(fn, A, B):
        M, K = A.shape
        N = B.shape[1]
        C = np.full((M, N), np.nan, np.float32)
        fn(ctypes.c_void_p(A.ctypes.data), ctypes.c_void_p(B.ctypes.data), ctypes.c_void_p(C.ctypes.data),
           i64(M), i64(N), i64(K))
        return C

    out = {}
    rng = np.random.default_rng(20240607)
    shapes = [(2, 2, 2), (4, 4, 4), (32, 32, 32), (65, 33, 17), (128, 96, 200), (1, 257, 63), (130, 1, 129)]
    for idx, (M, N, K) in enumerate(shapes):
        A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
        out[f"mm{idx}_A"] = A
        out[f"mm{idx}_B"] = B
        out[f"mm{idx}_py_matmul_jit"] = np.asarray(symplex.matmul_jit(A, B)._data, dtype=np.float32)
        out[f"mm{idx}_py_matmul_tiled"] = np.asarray(symplex.matmul_tiled(A, B)._data, dtype=np.float32)
        out[f"mm{idx}_c_matmul_f32"] = c_matmul(ref_c.symplex_matmul_f32, A, B)
        out[f"mm{idx}_c_matmul_tiled_f32"] = c_matmul(ref_c.symplex_matmul_tiled_f32, A, B)
    out["mm_count"] = np.int64(len(shapes))

    # The reference's own 2x2 known answer (python/tests/test_jit.py:60-66) through its API.
    A = np.array([[1, 2], [3, 4]], np.float32)
    B = np.array([[5, 6], [7, 8]], np.float32)
    out["kat2x2"] = np.asarray(symplex.matmul_jit(A, B)._data, dtype=np.float32)

    # Activations as the reference evaluates them (DeviceArray methods, python/symplex/_array.py:355-363).
    x = np.concatenate([np.linspace(-6, 6, 193), rng.normal(0, 1.5, 63)]).astype(np.float32)
    xa = symplex.array(x) if hasattr(symplex, "array") else symplex.DeviceArray(x)
    out["act_x"] = x
    out["act_gelu"] = np.asarray(xa.gelu()._data)
    out["act_relu"] = np.asarray(xa.relu()._data)
    out["act_sigmoid"] = np.asarray(xa.sigmoid()._data)
    out["act_tanh"] = np.asarray(xa.tanh()._data)

    # Fused chain through the reference's Python ops: gelu(X @ W + b), relu(X @ W + b).
    X = rng.normal(0, 0.5, (48, 40)).astype(np.float32)
    W = rng.normal(0, 0.5, (40, 56)).astype(np.float32)
    b = rng.normal(0, 0.5, 56).astype(np.float32)
    lin = symplex.DeviceArray(np.asarray(symplex.matmul_jit(X, W)._data) + b)
    out["fused_X"], out["fused_W"], out["fused_b"] = X, W, b
    out["fused_gelu"] = np.asarray(lin.gelu()._data, dtype=np.float32)
    out["fused_relu"] = np.asarray(lin.relu()._data, dtype=np.float32)

    # Fused elementwise chains through @symplex.jit (NumPy executor). n = 1003: not a multiple of 8, so the
    # interpreter's vector body and scalar tail are both exercised, and max / min meet the reference's tail rule.
    import contextlib
    import io
    n = 1003
    for tag, dt in (("f32", np.float32), ("f64", np.float64)):
        x, a, b, c = (rng.uniform(-1, 1, n).astype(dt) for _ in range(4))
        pos = rng.uniform(0.1, 3.0, n).astype(dt)
        out[f"fe_{tag}_x"], out[f"fe_{tag}_a"], out[f"fe_{tag}_b"], out[f"fe_{tag}_c"] = x, a, b, c
        out[f"fe_{tag}_pos"] = pos

        def run(fn, *args):
            with contextlib.redirect_stdout(io.StringIO()), contextlib.redirect_stderr(io.StringIO()):
                r = symplex.jit(fn)(*args)
            return np.asarray(getattr(r, "_data", r))

        out[f"fe_{tag}_axpb"] = run(lambda x: x * 2.0 + 1.0, x)
        out[f"fe_{tag}_axpb_sum"] = np.float64(run(lambda x: (x * 2.0 + 1.0).sum(), x))
        out[f"fe_{tag}_mul_add_relu"] = run(lambda a, b, c: symplex.relu(a * b + c), a, b, c)
        out[f"fe_{tag}_sub_div"] = run(lambda a, b, pos: (a - b) / pos, a, b, pos)
        out[f"fe_{tag}_libm"] = run(lambda x, pos: symplex.tanh(symplex.exp(x) * symplex.sqrt(pos)) + symplex.sigmoid(x),
                                    x, pos)
        out[f"fe_{tag}_max"] = np.float64(run(lambda a, b: (a * b).max(), a, b))
        out[f"fe_{tag}_min"] = np.float64(run(lambda a, b: (a + b).min(), a, b))

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
