/*
 * CPU ORACLE — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the arithmetic of SympleX's CPU matmul path, used only by the tests,
 * the smoke check and the benchmark's cpu_baseline / reference arm to check and to time against.
 * Nothing in the shipped library links, loads or calls this file.
 *
 * The reference's executable matmul lives in Rust (rust-engine/src/x86_emitter.rs) and cannot be
 * built where this was written (no rustc), so each function below restates, element by element and
 * rounding by rounding, what the machine code emitted by the reference computes. IEEE-754 fp32
 * fused multiply-add is fmaf(); separately rounded multiply and add are written as two statements
 * and this file must be compiled with -ffp-contract=off so the compiler keeps them apart.
 *
 * Pinning: checked by tests/test_oracle.py against every known-answer vector the reference's own
 * tests hold for this path (2x2 product, I4.B = B, the (7i+13)%97 / (11i+17)%89 pattern against a
 * scalar triple loop, gelu(0)=0) and against the reference's own kernels/matmul.c compiled unchanged
 * into oracle/_ref/. The fused elementwise chain (last section) has no vector in the reference's tests
 * either: parity unpinned, restated from the Rust source. bf16-input, GELU-fused and batched results have no vector in the reference:
 * parity for those is unpinned by the reference and rests on this restatement alone.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* ---- row-parallel driver (pthreads) -------------------------------------------------------------
 * Rows of C are independent in every kernel below, so splitting rows over threads changes speed only,
 * never a result. It mirrors how the reference parallelises (rayon over row blocks,
 * rust-engine/src/x86_emitter.rs:1861). */
typedef void (*row_fn)(void* ctx, int64_t r0, int64_t r1);
typedef struct { row_fn fn; void* ctx; int64_t r0, r1; } row_job;
static void* row_thread(void* arg) {
  row_job* j = (row_job*)arg;
  j->fn(j->ctx, j->r0, j->r1);
  return NULL;
}
static void parallel_rows(row_fn fn, void* ctx, int64_t rows, int threads) {
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  if ((int64_t)threads > rows) threads = rows > 0 ? (int)rows : 1;
  if (threads == 1) { fn(ctx, 0, rows); return; }
  pthread_t tid[256];
  row_job job[256];
  int started = 0;
  for (int t = 0; t < threads; ++t) {
    job[t].fn = fn; job[t].ctx = ctx;
    job[t].r0 = rows * t / threads;
    job[t].r1 = rows * (t + 1) / threads;
    if (t == threads - 1 || pthread_create(&tid[t], NULL, row_thread, &job[t]) != 0) {
      /* last slice (or a failed spawn) runs here, covering everything that is left */
      job[t].r1 = rows;
      fn(ctx, job[t].r0, job[t].r1);
      break;
    }
    ++started;
  }
  for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
}
typedef struct { const float* A; const float* B; float* C; int64_t M, N, K; const int64_t* rows; } mm_ctx;

/* ---- the AVX-512 size-baked JIT kernel --------------------------------------------------------
 * rust-engine/src/x86_emitter.rs:437-631 (compile_matmul_avx512):
 *   columns j < 16*floor(N/16): acc = 0; for k ascending: acc = fma(A[i,k], B[k,j], acc)
 *     (vfmadd231ps on 64-column blocks :487-551 and on 16-column blocks :554-577 - same per-element
 *      arithmetic, every lane is an independent k-sequential FMA chain);
 *   the last N mod 16 columns :580-617: acc = 0; for k: t = A[i,k]*B[k,j] (mulss); acc = acc + t (addss).
 * Rows are independent; `threads` only splits rows for speed and never changes a result. */
static void jit_order_rows(void* vctx, int64_t r0, int64_t r1) {
  const mm_ctx* x = (const mm_ctx*)vctx;
  const float* A = x->A; const float* B = x->B; float* C = x->C;
  const int64_t N = x->N, K = x->K;
  const int64_t n_fma = (N / 16) * 16;
  for (int64_t i = r0; i < r1; ++i) {
    const float* a = A + i * K;
    float* c = C + i * N;
    /* blocks of 64 accumulators keep B rows streaming, as the kernel's 4 ZMM accumulators do */
    for (int64_t j0 = 0; j0 < n_fma; j0 += 64) {
      const int64_t w = (n_fma - j0) < 64 ? (n_fma - j0) : 64;
      float acc[64];
      for (int64_t j = 0; j < w; ++j) acc[j] = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        const float aik = a[k];
        const float* b = B + k * N + j0;
        for (int64_t j = 0; j < w; ++j) acc[j] = fmaf(aik, b[j], acc[j]);
      }
      for (int64_t j = 0; j < w; ++j) c[j0 + j] = acc[j];
    }
    for (int64_t j = n_fma; j < N; ++j) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        float t = B[k * N + j] * a[k];
        acc = acc + t;
      }
      c[j] = acc;
    }
  }
}
void oracle_matmul_jit_order(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                             int threads) {
  mm_ctx x = {A, B, C, M, N, K, NULL};
  parallel_rows(jit_order_rows, &x, M, threads);
}

/* ---- the BLIS-style blocked kernel ------------------------------------------------------------
 * rust-engine/src/x86_emitter.rs:1616-1875: MC = NC = KC = 128. For each KC block of k (ascending,
 * :1724) the micro-kernel builds p = fma chain from 0 over the block's k (:1658-1673) and then does
 * C = C + p (:1676-1700). C starts at 0 (:1852-1854). Packing, MR/NR edges and zero padding do not
 * change any element's arithmetic. Row blocks are independent (rayon, :1861). */
static void blis_order_rows(void* vctx, int64_t r0, int64_t r1) {
  const mm_ctx* x = (const mm_ctx*)vctx;
  const float* A = x->A; const float* B = x->B; float* C = x->C;
  const int64_t N = x->N, K = x->K;
  const int64_t KC = 128, NB = 128;
  for (int64_t i = r0; i < r1; ++i) {
    const float* a = A + i * K;
    float* c = C + i * N;
    for (int64_t j = 0; j < N; ++j) c[j] = 0.0f;
    for (int64_t j0 = 0; j0 < N; j0 += NB) {
      const int64_t w = (N - j0) < NB ? (N - j0) : NB;
      for (int64_t k0 = 0; k0 < K; k0 += KC) {
        const int64_t kc = (K - k0) < KC ? (K - k0) : KC;
        float p[128];
        for (int64_t j = 0; j < w; ++j) p[j] = 0.0f;
        for (int64_t k = 0; k < kc; ++k) {
          const float aik = a[k0 + k];
          const float* b = B + (k0 + k) * N + j0;
          for (int64_t j = 0; j < w; ++j) p[j] = fmaf(aik, b[j], p[j]);
        }
        for (int64_t j = 0; j < w; ++j) c[j0 + j] = c[j0 + j] + p[j];
      }
    }
  }
}
void oracle_matmul_blis_order(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                              int threads) {
  mm_ctx x = {A, B, C, M, N, K, NULL};
  parallel_rows(blis_order_rows, &x, M, threads);
}

/* ---- dispatcher ---------------------------------------------------------------------------------
 * rust-engine/src/x86_emitter.rs:1899-1919 (jit_parallel_matmul) on an AVX-512 host: the size-baked
 * JIT kernel when N >= 64, otherwise the BLIS-blocked kernel. Zero dimension: C is left untouched. */
void oracle_jit_parallel_matmul(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                                int threads) {
  if (M == 0 || N == 0 || K == 0) return;
  if (N >= 64)
    oracle_matmul_jit_order(A, B, C, M, N, K, threads);
  else
    oracle_matmul_blis_order(A, B, C, M, N, K, threads);
}

/* rust-engine/src/x86_emitter.rs:1877-1897 (parallel_matmul) on an AVX2-or-better host. */
void oracle_parallel_matmul(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                            int threads) {
  if (M == 0 || N == 0 || K == 0) return;
  oracle_matmul_blis_order(A, B, C, M, N, K, threads);
}

/* ---- fused MatMul + Bias + ReLU -----------------------------------------------------------------
 * rust-engine/src/x86_emitter.rs:634-770: C zeroed; i-k-j with C updated through memory.
 * The 8-wide loop runs while the byte offset is < 4N-32 (:690-691), i.e. for column blocks starting
 * below N-8: those columns use vfmadd231ps (one rounding); all later columns - always including the
 * last 8 - use mulss + addss (two roundings) (:703-716). Then C = max(C + bias[j], 0) (:722-759). */
void oracle_fused_matmul_bias_relu(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                                   const float* bias) {
  int64_t vec_end = 0;
  while (vec_end < N - 8) vec_end += 8;
  for (int64_t i = 0; i < M; ++i) {
    float* c = C + i * N;
    for (int64_t j = 0; j < N; ++j) c[j] = 0.0f;
    for (int64_t k = 0; k < K; ++k) {
      const float aik = A[i * K + k];
      const float* b = B + k * N;
      for (int64_t j = 0; j < vec_end; ++j) c[j] = fmaf(aik, b[j], c[j]);
      for (int64_t j = vec_end; j < N; ++j) {
        float t = b[j] * aik;
        c[j] = c[j] + t;
      }
    }
    for (int64_t j = 0; j < N; ++j) {
      float s = c[j] + bias[j];
      c[j] = s > 0.0f ? s : 0.0f;
    }
  }
}

/* ---- the plain C kernel ---------------------------------------------------------------------------
 * kernels/matmul.c:7-18: zero C, then i-k-j "C += a*b" with separately rounded multiply and add
 * (what the source says; the reference's own build may contract or reassociate under -ffast-math,
 * which is why oracle/_ref/ holds that file compiled as-is for comparison). */
void oracle_matmul_c_order(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
  for (int64_t i = 0; i < M * N; ++i) C[i] = 0.0f;
  for (int64_t i = 0; i < M; ++i)
    for (int64_t k = 0; k < K; ++k) {
      const float aik = A[i * K + k];
      for (int64_t j = 0; j < N; ++j) {
        float t = aik * B[k * N + j];
        C[i * N + j] = C[i * N + j] + t;
      }
    }
}

/* matmul_bench.rs:16-27 (scalar_matmul): i-j-k, sum += a*b in fp32, two roundings. */
void oracle_scalar_matmul(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      float sum = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        float t = A[i * K + k] * B[k * N + j];
        sum = sum + t;
      }
      C[i * N + j] = sum;
    }
}

/* ---- operand conversions ------------------------------------------------------------------------ */

/* fp32 -> bf16 with round-to-nearest-even, returned widened back to fp32 ("bf16-rounded inputs"). */
float oracle_bf16_round(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) { /* inf / nan: keep class */
    u &= 0xffff0000u;
    if ((u & 0x7fffffffu) == 0x7f800000u || (u & 0x007f0000u)) { /* inf, or nan with a kept payload bit */
    } else {
      u |= 0x00400000u;
    }
  } else {
    u += 0x7fffu + ((u >> 16) & 1u);
    u &= 0xffff0000u;
  }
  float r;
  memcpy(&r, &u, 4);
  return r;
}
void oracle_bf16_round_array(const float* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = oracle_bf16_round(in[i]);
}
/* bf16 bit patterns <-> fp32 */
void oracle_bf16_bits_to_f32(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t u = (uint32_t)in[i] << 16;
    memcpy(&out[i], &u, 4);
  }
}
void oracle_f32_to_bf16_bits(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    float r = oracle_bf16_round(in[i]);
    uint32_t u;
    memcpy(&u, &r, 4);
    out[i] = (uint16_t)(u >> 16);
  }
}

/* ---- epilogues ------------------------------------------------------------------------------------
 * Activations as the reference defines them, evaluated in fp32:
 *   relu    max(x, 0)                                         python/symplex/_array.py:355-356
 *   gelu    0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))   python/symplex/_array.py:358-360
 *   sigmoid 1 / (1 + exp(-x))                                 python/symplex/_array.py:362-363,
 *                                                             rust-engine/src/x86_emitter.rs:1991 (opcode 14)
 *   tanh    tanh(x)                                           rust-engine/src/x86_emitter.rs:1990 (opcode 13)
 *   silu    x * sigmoid(x)                                    (OpType::SiLU, rust-engine/src/fusion_engine.rs:261-266)
 * Order of the fused chain [MatMul, Mul, Add, act] (rust-engine/src/fusion_engine.rs:1611-1618):
 *   y = act(alpha * acc + beta * r + bias[j]). */
float oracle_activation(float x, int act) {
  switch (act) {
    case 1: return x > 0.0f ? x : 0.0f;
    case 2: {
      const float c = 0.7978845608028654f; /* sqrt(2/pi) */
      float u = c * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + tanhf(u));
    }
    case 3: return 1.0f / (1.0f + expf(-x));
    case 4: return tanhf(x);
    case 5: return x / (1.0f + expf(-x));
    default: return x;
  }
}

void oracle_epilogue(float* C, int64_t M, int64_t N, float alpha, float beta, const float* residual,
                     const float* bias, int act) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      float v = C[i * N + j] * alpha;
      if (residual) v += beta * residual[i * N + j];
      if (bias) v += bias[j];
      C[i * N + j] = oracle_activation(v, act);
    }
}

/* Selected rows of C = A.B in JIT order: row r of the output is row rows[r] of the full product.
 * Exact for a row-partitioned contraction; lets the tests check the large configurations on a
 * sample of rows in seconds. */
static void jit_order_selected(void* vctx, int64_t r0, int64_t r1) {
  const mm_ctx* x = (const mm_ctx*)vctx;
  for (int64_t r = r0; r < r1; ++r) {
    mm_ctx one = {x->A + x->rows[r] * x->K, x->B, x->C + r * x->N, 1, x->N, x->K, NULL};
    jit_order_rows(&one, 0, 1);
  }
}
void oracle_matmul_jit_order_rows(const float* A, const float* B, float* Crows, const int64_t* rows, int64_t nrows,
                                  int64_t N, int64_t K, int threads) {
  mm_ctx x = {A, B, Crows, nrows, N, K, rows};
  parallel_rows(jit_order_selected, &x, nrows, threads);
}

/* Host cores available to this process. */
/* ---- fused elementwise chain with optional reduction --------------------------------------------
 * Restates fused_elem_f32_avx2_core (rust-engine/src/x86_emitter.rs:2027-2351): the op chain is evaluated
 * per element with separately rounded fp32 operations (ops 0-5 are vaddps/vsubps/vmulps/vdivps/vminps/
 * vmaxps, ops 6-15 go lane by lane through apply_unop_f32, :1981-1996, i.e. libm). The reduction keeps the
 * reference's accumulator structure: four 8-lane fp32 accumulators over blocks of 32 elements (:2044-2166),
 * accumulator 0 for the remaining blocks of 8 (:2169-2233), an f64 scalar for the last n mod 8 elements
 * (:2236-2295), then acc0+acc1, +acc2, +acc3 and the three shuffle steps (:2298-2344), and finally
 * "result as f64 + scalar_acc" (:2347) - which for max / min with a tail ADDS the two partial extrema; the
 * restatement keeps that so it is the reference's answer, and `exact` = 1 asks for the true extremum instead.
 * Operand rules: input / constant index out of range reads 0.0; a reference to op j >= the current op
 * reads 0.0 here (the scalar tail's rule, :2239; the vector body would read a stale value). */
typedef struct {
  uint8_t op, lhs_src;
  uint16_t lhs_idx;
  uint8_t rhs_src, pad_;
  uint16_t rhs_idx;
} oracle_fused_op;

static float fe_unop(uint8_t op, float v) {
  switch (op) {
    case 6: return -v;
    case 7: return fabsf(v);
    case 8: return sqrtf(v);
    case 9: return expf(v);
    case 10: return logf(v);
    case 11: return sinf(v);
    case 12: return cosf(v);
    case 13: return tanhf(v);
    case 14: { float e = expf(-v); float d = 1.0f + e; return 1.0f / d; }
    case 15: return v > 0.0f ? v : 0.0f; /* f32::max(0.0): NaN -> 0 */
    default: return v;
  }
}

static float fe_element(const oracle_fused_op* ops, int64_t n_ops, const float* const* in, int64_t n_in,
                        const float* consts, int64_t n_consts, int64_t i, float* tmp) {
  for (int64_t o = 0; o < n_ops; ++o) {
    float v[2];
    for (int side = 0; side < 2; ++side) {
      const uint8_t src = side ? ops[o].rhs_src : ops[o].lhs_src;
      const uint16_t idx = side ? ops[o].rhs_idx : ops[o].lhs_idx;
      float x = 0.0f;
      if (src == 0) x = idx < n_in ? in[idx][i] : 0.0f;
      else if (src == 1) x = idx < n_consts ? consts[idx] : 0.0f;
      else if (src == 2) x = idx < o ? tmp[idx] : 0.0f;
      v[side] = x;
    }
    float r;
    if (ops[o].op >= 6) r = fe_unop(ops[o].op, v[0]);
    else switch (ops[o].op) {
      case 0: r = v[0] + v[1]; break;
      case 1: r = v[0] - v[1]; break;
      case 2: r = v[0] * v[1]; break;
      case 3: r = v[0] / v[1]; break;
      case 4: r = v[0] < v[1] ? v[0] : v[1]; break; /* vminps: second operand unless first is smaller */
      default: r = v[0] > v[1] ? v[0] : v[1]; break;
    }
    tmp[o] = r;
  }
  return tmp[n_ops - 1];
}

static float fe_red(int reduce_op, float a, float b) {
  if (reduce_op == 0) return a + b;
  if (reduce_op == 1) return a > b ? a : b; /* vmaxps(acc, v) */
  return a < b ? a : b;
}

double oracle_fused_elementwise_f32(const oracle_fused_op* ops, int64_t n_ops, const float* const* in, int64_t n_in,
                                    const float* consts, int64_t n_consts, int64_t n, int reduce_op, float* dst,
                                    int exact) {
  if (n <= 0 || n_ops <= 0) return 0.0;
  float* tmp = (float*)malloc(sizeof(float) * (size_t)n_ops);
  const int has_reduce = reduce_op != 255;
  const float init = reduce_op == 1 ? -INFINITY : reduce_op == 2 ? INFINITY : 0.0f;
  float acc[4][8];
  for (int a = 0; a < 4; ++a) for (int l = 0; l < 8; ++l) acc[a][l] = init;
  int64_t i = 0;
  const int64_t n32 = n & ~(int64_t)31, n8 = n & ~(int64_t)7;
  for (; i < n32; i += 32)
    for (int u = 0; u < 4; ++u)
      for (int l = 0; l < 8; ++l) {
        const int64_t e = i + u * 8 + l;
        const float v = fe_element(ops, n_ops, in, n_in, consts, n_consts, e, tmp);
        if (has_reduce) acc[u][l] = fe_red(reduce_op, acc[u][l], v);
        else dst[e] = v;
      }
  for (; i < n8; i += 8)
    for (int l = 0; l < 8; ++l) {
      const float v = fe_element(ops, n_ops, in, n_in, consts, n_consts, i + l, tmp);
      if (has_reduce) acc[0][l] = fe_red(reduce_op, acc[0][l], v);
      else dst[i + l] = v;
    }
  double scalar_acc = 0.0;
  int first = 1;
  for (; i < n; ++i) {
    const float v = fe_element(ops, n_ops, in, n_in, consts, n_consts, i, tmp);
    if (!has_reduce) { dst[i] = v; continue; }
    if (reduce_op == 0) scalar_acc += (double)v;
    else if (first) scalar_acc = (double)v;
    else if (reduce_op == 1) scalar_acc = scalar_acc > (double)v ? scalar_acc : (double)v;
    else scalar_acc = scalar_acc < (double)v ? scalar_acc : (double)v;
    first = 0;
  }
  free(tmp);
  if (!has_reduce) return 0.0;
  float a0[8];
  for (int l = 0; l < 8; ++l) {
    float t = fe_red(reduce_op, acc[0][l], acc[1][l]);
    t = fe_red(reduce_op, t, acc[2][l]);
    a0[l] = fe_red(reduce_op, t, acc[3][l]);
  }
  float s1[4], s2[2];
  for (int l = 0; l < 4; ++l) s1[l] = fe_red(reduce_op, a0[l], a0[l + 4]); /* swap 128-bit halves */
  for (int l = 0; l < 2; ++l) s2[l] = fe_red(reduce_op, s1[l], s1[l + 2]); /* shuffle 0x4E */
  const float r = fe_red(reduce_op, s2[0], s2[1]);                         /* shuffle 0xB1 */
  if (exact && reduce_op != 0) {
    if (first) return (double)r;      /* no tail */
    if (n8 == 0) return scalar_acc;   /* tail only */
    return reduce_op == 1 ? ((double)r > scalar_acc ? (double)r : scalar_acc)
                          : ((double)r < scalar_acc ? (double)r : scalar_acc);
  }
  return (double)r + scalar_acc;
}

/* The f64 twin, fused_elem_f64_avx2_core (rust-engine/src/x86_emitter.rs:2478-2727): same chain rules in double;
 * four 4-lane accumulators over blocks of 16, accumulator 0 for the remaining blocks of 4, a scalar for the last
 * n mod 4, then acc0+acc1, +acc2, +acc3, lanes l + (l+2), then lane 0 + lane 1, "+ scalar_acc". */
static double fe_unop64(uint8_t op, double v) {
  switch (op) {
    case 6: return -v;
    case 7: return fabs(v);
    case 8: return sqrt(v);
    case 9: return exp(v);
    case 10: return log(v);
    case 11: return sin(v);
    case 12: return cos(v);
    case 13: return tanh(v);
    case 14: return 1.0 / (1.0 + exp(-v));
    case 15: return v > 0.0 ? v : 0.0;
    default: return v;
  }
}

static double fe_element64(const oracle_fused_op* ops, int64_t n_ops, const double* const* in, int64_t n_in,
                           const double* consts, int64_t n_consts, int64_t i, double* tmp) {
  for (int64_t o = 0; o < n_ops; ++o) {
    double v[2];
    for (int side = 0; side < 2; ++side) {
      const uint8_t src = side ? ops[o].rhs_src : ops[o].lhs_src;
      const uint16_t idx = side ? ops[o].rhs_idx : ops[o].lhs_idx;
      double x = 0.0;
      if (src == 0) x = idx < n_in ? in[idx][i] : 0.0;
      else if (src == 1) x = idx < n_consts ? consts[idx] : 0.0;
      else if (src == 2) x = idx < o ? tmp[idx] : 0.0;
      v[side] = x;
    }
    double r;
    if (ops[o].op >= 6) r = fe_unop64(ops[o].op, v[0]);
    else switch (ops[o].op) {
      case 0: r = v[0] + v[1]; break;
      case 1: r = v[0] - v[1]; break;
      case 2: r = v[0] * v[1]; break;
      case 3: r = v[0] / v[1]; break;
      case 4: r = v[0] < v[1] ? v[0] : v[1]; break;
      default: r = v[0] > v[1] ? v[0] : v[1]; break;
    }
    tmp[o] = r;
  }
  return tmp[n_ops - 1];
}

static double fe_red64(int reduce_op, double a, double b) {
  if (reduce_op == 0) return a + b;
  if (reduce_op == 1) return a > b ? a : b;
  return a < b ? a : b;
}

double oracle_fused_elementwise_f64(const oracle_fused_op* ops, int64_t n_ops, const double* const* in, int64_t n_in,
                                    const double* consts, int64_t n_consts, int64_t n, int reduce_op, double* dst,
                                    int exact) {
  if (n <= 0 || n_ops <= 0) return 0.0;
  double* tmp = (double*)malloc(sizeof(double) * (size_t)n_ops);
  const int has_reduce = reduce_op != 255;
  const double init = reduce_op == 1 ? -INFINITY : reduce_op == 2 ? INFINITY : 0.0;
  double acc[4][4];
  for (int a = 0; a < 4; ++a) for (int l = 0; l < 4; ++l) acc[a][l] = init;
  int64_t i = 0;
  const int64_t n16 = n & ~(int64_t)15, n4 = n & ~(int64_t)3;
  for (; i < n16; i += 16)
    for (int u = 0; u < 4; ++u)
      for (int l = 0; l < 4; ++l) {
        const int64_t e = i + u * 4 + l;
        const double v = fe_element64(ops, n_ops, in, n_in, consts, n_consts, e, tmp);
        if (has_reduce) acc[u][l] = fe_red64(reduce_op, acc[u][l], v);
        else dst[e] = v;
      }
  for (; i < n4; i += 4)
    for (int l = 0; l < 4; ++l) {
      const double v = fe_element64(ops, n_ops, in, n_in, consts, n_consts, i + l, tmp);
      if (has_reduce) acc[0][l] = fe_red64(reduce_op, acc[0][l], v);
      else dst[i + l] = v;
    }
  double scalar_acc = 0.0;
  int first = 1;
  for (; i < n; ++i) {
    const double v = fe_element64(ops, n_ops, in, n_in, consts, n_consts, i, tmp);
    if (!has_reduce) { dst[i] = v; continue; }
    if (reduce_op == 0) scalar_acc += v;
    else if (first) scalar_acc = v;
    else scalar_acc = fe_red64(reduce_op, scalar_acc, v);
    first = 0;
  }
  free(tmp);
  if (!has_reduce) return 0.0;
  double a0[4];
  for (int l = 0; l < 4; ++l) {
    double t = fe_red64(reduce_op, acc[0][l], acc[1][l]);
    t = fe_red64(reduce_op, t, acc[2][l]);
    a0[l] = fe_red64(reduce_op, t, acc[3][l]);
  }
  const double s0 = fe_red64(reduce_op, a0[0], a0[2]), s1 = fe_red64(reduce_op, a0[1], a0[3]);
  const double r = fe_red64(reduce_op, s0, s1);
  if (exact && reduce_op != 0) {
    if (first) return r;
    if (n4 == 0) return scalar_acc;
    return fe_red64(reduce_op, r, scalar_acc);
  }
  return r + scalar_acc;
}

/* ---- the f64 tiled GEMM behind blas_dgemm / cache_tiled_dgemm_thin ------------------------------
 * rust-engine/src/phase3_jit.rs:578-650 (cache_tiled_dgemm): C = 0; for each block of KC = 128 consecutive k
 * (ascending): acc = 0; for k in the block: acc = acc + a*b - Rust rounds the product and the sum separately
 * (no contraction; this file is compiled with -ffp-contract=off) - then C = C + acc. The MC / NC / MR / NR
 * tiling and the packing only reorder which elements are worked on, never an element's own arithmetic.
 * Unpinned by the reference's tests (none calls it); pinned here only through the structure above. */
void oracle_cache_tiled_dgemm(const double* A, const double* B, double* C, int64_t M, int64_t N, int64_t K) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      double c = 0.0;
      for (int64_t k0 = 0; k0 < K; k0 += 128) {
        const int64_t k1 = k0 + 128 < K ? k0 + 128 : K;
        double acc = 0.0;
        for (int64_t k = k0; k < k1; ++k) {
          double t = A[i * K + k] * B[k * N + j];
          acc = acc + t;
        }
        c = c + acc;
      }
      C[i * N + j] = c;
    }
}

int oracle_max_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}
