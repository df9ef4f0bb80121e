/*
 * CPU ORACLE — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * AVX-512 restatement of the reference's size-baked JIT matmul kernel, instruction for instruction where the
 * arithmetic is concerned (rust-engine/src/x86_emitter.rs:437-631, compile_matmul_avx512):
 *   for i in 0..M
 *     for each block of 64 columns (:487-551):  zmm acc0..acc3 = 0
 *        for k in 0..K: a = vbroadcastss A[i,k];  acc_t = vfmadd231ps(a, B[k, j+16t .. j+16t+15], acc_t)   t = 0..3
 *        store acc0..acc3 to C[i, j..j+63]
 *     for each remaining block of 16 columns (:554-577): the same with one accumulator
 *     for each of the last N mod 16 columns (:580-617): acc = 0; for k: t = mulss(B[k,j], A[i,k]); acc = addss(acc, t)
 * It is the metric's own CPU comparator ("CPU x86-JIT"): single-threaded, like the reference's AVX-512 path
 * (x86_emitter.rs:1904-1910), timed by the benchmark on one host core. tests/test_oracle.py checks that it returns
 * the bits of the scalar restatement oracle_matmul_jit_order (every lane is the same k-sequential fp32 FMA chain).
 * Built into liboracle.so; the functions carry their own target attribute and the entry point checks the CPU, so
 * the library loads on hosts without AVX-512 (the entry point then returns -1 and nothing is computed).
 */
#include <immintrin.h>
#include <stdint.h>

__attribute__((target("avx512f"))) static void jit_avx512_rows(const float* A, const float* B, float* C, int64_t M,
                                                                int64_t N, int64_t K) {
  const int64_t n64 = N / 64, n16 = (N % 64) / 16;
  for (int64_t i = 0; i < M; ++i) {
    const float* a = A + i * K;
    float* c = C + i * N;
    int64_t j = 0;
    for (int64_t jb = 0; jb < n64; ++jb, j += 64) {
      __m512 acc0 = _mm512_setzero_ps(), acc1 = _mm512_setzero_ps(), acc2 = _mm512_setzero_ps(),
             acc3 = _mm512_setzero_ps();
      const float* b = B + j;
      for (int64_t k = 0; k < K; ++k, b += N) {
        const __m512 av = _mm512_set1_ps(a[k]);
        acc0 = _mm512_fmadd_ps(av, _mm512_loadu_ps(b), acc0);
        acc1 = _mm512_fmadd_ps(av, _mm512_loadu_ps(b + 16), acc1);
        acc2 = _mm512_fmadd_ps(av, _mm512_loadu_ps(b + 32), acc2);
        acc3 = _mm512_fmadd_ps(av, _mm512_loadu_ps(b + 48), acc3);
      }
      _mm512_storeu_ps(c + j, acc0);
      _mm512_storeu_ps(c + j + 16, acc1);
      _mm512_storeu_ps(c + j + 32, acc2);
      _mm512_storeu_ps(c + j + 48, acc3);
    }
    for (int64_t jb = 0; jb < n16; ++jb, j += 16) {
      __m512 acc = _mm512_setzero_ps();
      const float* b = B + j;
      for (int64_t k = 0; k < K; ++k, b += N) acc = _mm512_fmadd_ps(_mm512_set1_ps(a[k]), _mm512_loadu_ps(b), acc);
      _mm512_storeu_ps(c + j, acc);
    }
    for (; j < N; ++j) {
      __m128 acc = _mm_setzero_ps();
      for (int64_t k = 0; k < K; ++k) acc = _mm_add_ss(acc, _mm_mul_ss(_mm_load_ss(B + k * N + j), _mm_load_ss(a + k)));
      _mm_store_ss(c + j, acc);
    }
  }
}

/* 0: computed; -1: this CPU has no AVX-512F (nothing is written). */
int oracle_matmul_jit_avx512(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
  if (!__builtin_cpu_supports("avx512f")) return -1;
  jit_avx512_rows(A, B, C, M, N, K);
  return 0;
}
