// Fused elementwise programs with an optional reduction, as one streaming pass over HBM.
//
// Replaces the reference's single-pass AVX2 interpreter for FusedOpDesc chains
// (rust-engine/src/x86_emitter.rs:1937-2351, entry point simd_fused_elementwise_f32 at :2442-2470) and the
// elementwise / fma / reduction kernels its PTX generator emits (rust-engine/src/cuda_backend.rs:220-694).
// A program is a list of ops; each op reads two operands (an input array, a constant, or the result of an
// earlier op) and produces one value per element. The last op's value is either stored to dst or reduced
// (sum / max / min) to one scalar.
//
// The kernel is HBM-bound: every input element is read exactly once and every output element written once.
// A producer thread streams 4 or 8 KB chunks of each input into a shared-memory ring with bulk async copies
// (mbarrier completion), so the bytes in flight per SM are set by the ring size, not by registers; 256
// consumer threads interpret the program out of the kernel's parameter block (constant bank, warp-uniform
// control flow) on float4 vectors read from the ring and store results with 16-byte coalesced stores.
// Values that are consumed by the very next op stay in registers; values with a longer life go to a small
// per-thread slot file whose slots the host assigns by liveness. Arrays that are not 16-byte aligned take a
// plain-load variant of the same interpreter.
//
// Arithmetic follows the reference op by op: add / sub / mul / div are separately rounded IEEE operations
// (never contracted into FMAs), sqrt is correctly rounded, min / max follow the AVX2 forms
// (l < r ? l : r and l > r ? l : r). exp, log, sin, cos, tanh use CUDA's libm (<= 2 ulp).
// Everything is templated on the element type: float (simd_fused_elementwise_f32) and double (the _f64 twin).
#include <cstring>
#include <memory>
#include <vector>

#include "gemm_params.h"
#include "host_api.h"
#include "sm100_ptx.cuh"

namespace sx {

// ------------------------------------------------------------------------------------------------ host compile
int compile_fused_program(const FeSrcOp* ops, size_t n_ops, size_t n_inputs, const void* constants,
                          size_t n_constants, int elem_bytes, FeProgram* out) {
  if (ops == nullptr || n_ops == 0) return set_last_error(SX_ERR_INVALID, "empty program");
  if (elem_bytes != 4 && elem_bytes != 8) return set_last_error(SX_ERR_INVALID, "element size must be 4 or 8");
  if (n_ops > (size_t)FE_MAX_OPS) return set_last_error(SX_ERR_INVALID, "program has more than 1024 ops");
  if (n_constants && constants == nullptr) return set_last_error(SX_ERR_INVALID, "null constants");
  enum : uint8_t { REF = 200 };  // temporary kind: result of an earlier op
  struct Operand {
    uint8_t kind;
    uint64_t v;
  };
  FeProgram& P = *out;
  P.n_ops = (int)n_ops;
  P.n_inputs = 0;
  P.n_slots = 0;
  std::vector<int> compact;  // caller's input index -> compacted index, filled on first use
  auto resolve = [&](uint8_t src, uint16_t idx, size_t i, int* err) -> Operand {
    if (src == 0) {
      if (idx >= n_inputs) return {FE_IMM, 0u};  // the reference substitutes zero
      if (compact.empty()) compact.assign(n_inputs < 65536 ? n_inputs : 65536, -1);
      if (compact[idx] < 0) {
        if (P.n_inputs == FE_MAX_INPUTS) {
          *err = 1;
          return {FE_IMM, 0u};
        }
        compact[idx] = P.n_inputs;
        P.input_map[P.n_inputs++] = idx;
      }
      return {FE_IN, (uint64_t)compact[idx]};
    }
    if (src == 1) {
      uint64_t bits = 0;  // a float's bits sit in the low word
      if (idx < n_constants) memcpy(&bits, static_cast<const char*>(constants) + (size_t)idx * elem_bytes, elem_bytes);
      return {FE_IMM, bits};
    }
    if (src == 2 && idx < i) return {REF, idx};
    return {FE_IMM, 0u};  // forward references and unknown sources read as zero
  };
  std::vector<Operand> L(n_ops), R(n_ops);
  std::vector<int> last_use(n_ops, -1), slot_of(n_ops, -1);
  int err = 0;
  for (size_t i = 0; i < n_ops; ++i) {
    const bool unary = ops[i].op >= 6;
    L[i] = resolve(ops[i].lhs_src, ops[i].lhs_idx, i, &err);
    R[i] = unary ? Operand{FE_IMM, 0u} : resolve(ops[i].rhs_src, ops[i].rhs_idx, i, &err);
    if (L[i].kind == REF) last_use[L[i].v] = (int)i;
    if (R[i].kind == REF) last_use[R[i].v] = (int)i;
  }
  if (err) return set_last_error(SX_ERR_INVALID, "program reads more than 16 distinct input arrays");
  int free_slots[FE_MAX_SLOTS], n_free = 0;
  for (size_t i = 0; i < n_ops; ++i) {
    FeOp& o = P.ops[i];
    o.opcode = ops[i].op <= 15 ? ops[i].op : 16;  // 16: pass the left operand through
    auto lower = [&](const Operand& x, uint8_t* kind, uint64_t* v) {
      if (x.kind != REF) {
        *kind = x.kind;
        *v = x.v;
      } else if (x.v + 1 == i) {
        *kind = FE_LAST;
        *v = 0;
      } else {
        *kind = FE_SLOT;
        *v = (uint64_t)slot_of[x.v];
      }
    };
    lower(L[i], &o.lkind, &o.l);
    lower(R[i], &o.rkind, &o.r);
    // Slots whose value dies here can already take this op's result: operands are read before the write.
    auto release = [&](const Operand& x) {
      if (x.kind == REF && last_use[x.v] == (int)i && slot_of[x.v] >= 0) {
        free_slots[n_free++] = slot_of[x.v];
        slot_of[x.v] = -1;
      }
    };
    release(L[i]);
    release(R[i]);
    o.dst = FE_NO_DST;
    if (last_use[i] > (int)i + 1) {  // used beyond the next op: needs a slot
      int s;
      if (n_free > 0) {
        s = free_slots[--n_free];
      } else if (P.n_slots < FE_MAX_SLOTS) {
        s = P.n_slots++;
      } else {
        return set_last_error(SX_ERR_INVALID, "program keeps more than 16 intermediate values alive at once");
      }
      slot_of[i] = s;
      o.dst = (uint8_t)s;
    }
  }
  return SX_OK;
}

// ------------------------------------------------------------------------------------------------ device side
constexpr int FE_THREADS = 256;  // consumer threads; the ring kernel adds one producer warp
constexpr int FE_MAX_STAGES = 16;

template <typename T, int MAXOPS>
struct FeKernelArgs {
  long long n;
  const T* in[FE_MAX_INPUTS];
  T* dst;
  double* partials;
  unsigned* ticket;
  double* result;
  int* status;
  int n_ops, reduce_op, n_inputs, stages;
  int head;  // ring kernel: elements in front of element 0 (at indices -head .. -1) that belong to the arrays too
  FeOp ops[MAXOPS];
};

// Per-type arithmetic: explicitly rounded intrinsics so that nothing is contracted into an FMA.
template <typename T>
struct FeMath;
template <>
struct FeMath<float> {
  static constexpr int VE = 4;  // elements per 16-byte vector
  __device__ static float imm(uint64_t bits) { return __uint_as_float((uint32_t)bits); }
  __device__ static float add(float a, float b) { return __fadd_rn(a, b); }
  __device__ static float sub(float a, float b) { return __fsub_rn(a, b); }
  __device__ static float mul(float a, float b) { return __fmul_rn(a, b); }
  __device__ static float div(float a, float b) { return __fdiv_rn(a, b); }
  __device__ static float sqrt(float a) { return __fsqrt_rn(a); }
  __device__ static float abs(float a) { return fabsf(a); }
  __device__ static float exp(float a) { return expf(a); }
  __device__ static float log(float a) { return logf(a); }
  __device__ static float sin(float a) { return sinf(a); }
  __device__ static float cos(float a) { return cosf(a); }
  __device__ static float tanh(float a) { return tanhf(a); }
  __device__ static float max(float a, float b) { return fmaxf(a, b); }
  __device__ static float min(float a, float b) { return fminf(a, b); }
  __device__ static float inf() { return INFINITY; }
  __device__ static void load16(const float* p, float (&o)[4]) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    o[0] = q.x, o[1] = q.y, o[2] = q.z, o[3] = q.w;
  }
  __device__ static void store16_streaming(float* p, const float (&v)[4]) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
  }
  __device__ static void pin(float a) { asm volatile("" ::"f"(a) : "memory"); }
};
template <>
struct FeMath<double> {
  static constexpr int VE = 2;
  __device__ static double imm(uint64_t bits) { return __longlong_as_double((long long)bits); }
  __device__ static double add(double a, double b) { return __dadd_rn(a, b); }
  __device__ static double sub(double a, double b) { return __dsub_rn(a, b); }
  __device__ static double mul(double a, double b) { return __dmul_rn(a, b); }
  __device__ static double div(double a, double b) { return __ddiv_rn(a, b); }
  __device__ static double sqrt(double a) { return __dsqrt_rn(a); }
  __device__ static double abs(double a) { return fabs(a); }
  __device__ static double exp(double a) { return ::exp(a); }
  __device__ static double log(double a) { return ::log(a); }
  __device__ static double sin(double a) { return ::sin(a); }
  __device__ static double cos(double a) { return ::cos(a); }
  __device__ static double tanh(double a) { return ::tanh(a); }
  __device__ static double max(double a, double b) { return fmax(a, b); }
  __device__ static double min(double a, double b) { return fmin(a, b); }
  __device__ static double inf() { return (double)INFINITY; }
  __device__ static void load16(const double* p, double (&o)[2]) {
    const double2 q = *reinterpret_cast<const double2*>(p);
    o[0] = q.x, o[1] = q.y;
  }
  __device__ static void store16_streaming(double* p, const double (&v)[2]) {
    __stcs(reinterpret_cast<double2*>(p), make_double2(v[0], v[1]));
  }
  __device__ static void pin(double a) { asm volatile("" ::"d"(a) : "memory"); }
};

// Unary ops (and the pass-through for unknown codes) on W values.
template <typename T, int W>
__device__ __forceinline__ void fe_unary(uint32_t opcode, const T (&l)[W], T (&o)[W]) {
  using M = FeMath<T>;
  switch (opcode) {
#define FE_CASE(code, expr)                         \
  case code:                                        \
    _Pragma("unroll") for (int w = 0; w < W; ++w) { \
      const T a = l[w];                             \
      o[w] = (expr);                                \
    }                                               \
    break;
    FE_CASE(6, -a)
    FE_CASE(7, M::abs(a))
    FE_CASE(8, M::sqrt(a))
    FE_CASE(9, M::exp(a))
    FE_CASE(10, M::log(a))
    FE_CASE(11, M::sin(a))
    FE_CASE(12, M::cos(a))
    FE_CASE(13, M::tanh(a))
    FE_CASE(14, M::div(T(1), M::add(T(1), M::exp(-a))))
    FE_CASE(15, M::max(a, T(0)))
#undef FE_CASE
    default:
#pragma unroll
      for (int w = 0; w < W; ++w) o[w] = l[w];
      break;
  }
}

// The six exactly rounded binary ops on operand accessors (callables w -> value). `out` may be the array an
// accessor reads: element w is read before it is written.
template <typename T, int W, class LF, class RF>
__device__ __forceinline__ void fe_binary(uint32_t opcode, LF lf, RF rf, T (&out)[W]) {
  using M = FeMath<T>;
  switch (opcode) {
#define FE_BIN(code, expr)                          \
  case code:                                        \
    _Pragma("unroll") for (int w = 0; w < W; ++w) { \
      const T a = lf(w), b = rf(w);                 \
      out[w] = (expr);                              \
    }                                               \
    break;
    FE_BIN(0, M::add(a, b))
    FE_BIN(1, M::sub(a, b))
    FE_BIN(2, M::mul(a, b))
    FE_BIN(3, M::div(a, b))
    FE_BIN(4, (a < b) ? a : b)
    default:
      FE_BIN(5, (a > b) ? a : b)
#undef FE_BIN
  }
}

// Input loaders: hand the interpreter W values of input `idx` for this thread.
template <typename T, int U>
struct RingLoader {  // 16-byte vectors out of one ring stage; input i starts at base + i * stride
  static constexpr int VE = FeMath<T>::VE;
  const T* base;
  int stride;
  __device__ __forceinline__ void load(uint32_t idx, T (&o)[U * VE]) const {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      T q[VE];
      FeMath<T>::load16(base + (size_t)idx * stride + u * (FE_THREADS * VE), q);
#pragma unroll
      for (int k = 0; k < VE; ++k) o[u * VE + k] = q[k];
    }
  }
};
template <typename T, int U>
struct GlobalLoader {  // scalars straight from global memory at element offsets e[u]
  const T* const* in;
  long long e[U];
  bool ok[U];
  __device__ __forceinline__ void load(uint32_t idx, T (&o)[U]) const {
    const T* p = in[idx];
#pragma unroll
    for (int u = 0; u < U; ++u) o[u] = ok[u] ? __ldg(p + e[u]) : T(0);
  }
};

// Interpret the program for W values per thread; the last op's values end up in `last`.
// Binary arithmetic ops are dispatched on (left kind, right kind, opcode) to loops that read their operands
// in place - registers of `last`, an immediate, a slot, or freshly loaded input values - so an op costs one
// arithmetic instruction per element plus a warp-uniform dispatch; unary ops copy their operand first.
template <typename T, int W, int MAXOPS, class Loader>
__device__ __forceinline__ void fe_eval(const FeKernelArgs<T, MAXOPS>& P, const Loader& ld, T (&last)[W]) {
  using M = FeMath<T>;
  T slots[FE_MAX_SLOTS][W];
#pragma unroll
  for (int w = 0; w < W; ++w) last[w] = T(0);
  for (int i = 0; i < P.n_ops; ++i) {
    const FeOp op = P.ops[i];
    if (op.opcode < 6) {
      auto with_left = [&](auto lf) {
        switch (op.rkind) {
          case FE_IMM: {
            const T c = M::imm(op.r);
            fe_binary<T, W>(op.opcode, lf, [=](int) { return c; }, last);
          } break;
          case FE_LAST:
            fe_binary<T, W>(op.opcode, lf, [&](int w) { return last[w]; }, last);
            break;
          case FE_SLOT:
            fe_binary<T, W>(op.opcode, lf, [&](int w) { return slots[op.r][w]; }, last);
            break;
          default: {
            T t[W];
            ld.load((uint32_t)op.r, t);
            fe_binary<T, W>(op.opcode, lf, [&](int w) { return t[w]; }, last);
          } break;
        }
      };
      switch (op.lkind) {
        case FE_IMM: {
          const T c = M::imm(op.l);
          with_left([=](int) { return c; });
        } break;
        case FE_LAST:
          with_left([&](int w) { return last[w]; });
          break;
        case FE_SLOT:
          with_left([&](int w) { return slots[op.l][w]; });
          break;
        default: {
          T t[W];
          ld.load((uint32_t)op.l, t);
          with_left([&](int w) { return t[w]; });
        } break;
      }
    } else {
      T l[W];
      if (op.lkind == FE_IN) {
        ld.load((uint32_t)op.l, l);
      } else if (op.lkind == FE_IMM) {
#pragma unroll
        for (int w = 0; w < W; ++w) l[w] = M::imm(op.l);
      } else if (op.lkind == FE_LAST) {
#pragma unroll
        for (int w = 0; w < W; ++w) l[w] = last[w];
      } else {
#pragma unroll
        for (int w = 0; w < W; ++w) l[w] = slots[op.l][w];
      }
      fe_unary<T, W>(op.opcode, l, last);
    }
    if (op.dst != FE_NO_DST) {
#pragma unroll
      for (int w = 0; w < W; ++w) slots[op.dst][w] = last[w];
    }
  }
}

template <typename T>
__device__ __forceinline__ T fe_identity(int reduce_op) {
  return reduce_op == 1 ? -FeMath<T>::inf() : reduce_op == 2 ? FeMath<T>::inf() : T(0);
}
__device__ __forceinline__ double fe_combine(int reduce_op, double a, double b) {
  return reduce_op == 0 ? a + b : reduce_op == 1 ? fmax(a, b) : fmin(a, b);
}

// acc[w] = combine(acc[w], v[w]) with the choice of the operation hoisted out of the element loop.
template <typename T, int W>
__device__ __forceinline__ void fe_accumulate(int reduce_op, T (&acc)[W], const T (&v)[W]) {
  using M = FeMath<T>;
  if (reduce_op == 0) {
#pragma unroll
    for (int w = 0; w < W; ++w) acc[w] = M::add(acc[w], v[w]);
  } else if (reduce_op == 1) {
#pragma unroll
    for (int w = 0; w < W; ++w) acc[w] = M::max(acc[w], v[w]);
  } else {
#pragma unroll
    for (int w = 0; w < W; ++w) acc[w] = M::min(acc[w], v[w]);
  }
}

// Block-wide reduction in a fixed order; every thread of the block must call it. Result valid in thread 0.
__device__ __forceinline__ double fe_block_reduce(int reduce_op, double v, double* smem) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fe_combine(reduce_op, v, __shfl_xor_sync(0xffffffffu, v, off));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    v = lane < nw ? smem[lane] : fe_identity<double>(reduce_op);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fe_combine(reduce_op, v, __shfl_xor_sync(0xffffffffu, v, off));
  }
  return v;
}

// Fold the per-thread accumulators of the whole grid into *P.result: per block in a fixed order, then the
// block that arrives last folds the per-block partials in index order - the same bits on every run.
template <typename T, int W, int MAXOPS>
__device__ __forceinline__ void fe_grid_reduce(const FeKernelArgs<T, MAXOPS>& P, const T (&acc)[W]) {
  __shared__ double red[32];
  __shared__ bool is_last;
  double v = (double)acc[0];
#pragma unroll
  for (int w = 1; w < W; ++w) v = fe_combine(P.reduce_op, v, (double)acc[w]);
  v = fe_block_reduce(P.reduce_op, v, red);
  if (threadIdx.x == 0) {
    P.partials[blockIdx.x] = v;
    __threadfence();
    is_last = atomicAdd(P.ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    double s = fe_identity<double>(P.reduce_op);
    for (unsigned i = threadIdx.x; i < gridDim.x; i += blockDim.x) s = fe_combine(P.reduce_op, s, __ldcg(P.partials + i));
    s = fe_block_reduce(P.reduce_op, s, red);
    if (threadIdx.x == 0) {
      *P.result = s;
      *P.ticket = 0u;
    }
  }
}

// Elements [first, n) one per thread with plain loads: what is left after the last full chunk - and, behind them in
// the same loop, the P.head elements in front of element 0 (arrays that start a few elements before a 16-byte
// boundary are handed to the ring kernel from that boundary on).
template <typename T, int MAXOPS>
__device__ __forceinline__ void fe_scalar_range(const FeKernelArgs<T, MAXOPS>& P, long long first, long long gtid,
                                                long long nthreads, bool reduce, T& acc) {
  for (long long i = first + gtid; i < P.n + P.head; i += nthreads) {
    const long long t = i < P.n ? i : i - P.n - P.head;  // -head .. -1
    GlobalLoader<T, 1> ld;
    ld.in = P.in;
    ld.e[0] = t;
    ld.ok[0] = true;
    T r1[1], a1[1] = {acc};
    fe_eval<T, 1, MAXOPS>(P, ld, r1);
    if (reduce) {
      fe_accumulate<T, 1>(P.reduce_op, a1, r1);
      acc = a1[0];
    } else {
      P.dst[t] = r1[0];
    }
  }
}

// Ring kernel. Shared memory: [0,128) full barriers, [128,256) empty barriers, then `stages` stages of
// n_inputs x CHUNK elements (16 bytes x U per consumer thread). Chunk c of the arrays goes to CTA c mod gridDim.x.
template <typename T, int U, int MAXOPS>
__global__ void __launch_bounds__(FE_THREADS + 32)
fused_elementwise_ring_kernel(const __grid_constant__ FeKernelArgs<T, MAXOPS> P) {
  constexpr int VE = FeMath<T>::VE;
  constexpr int W = U * VE;
  constexpr int CHUNK = FE_THREADS * W;  // elements per input per stage
  extern __shared__ __align__(128) uint8_t fe_smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(fe_smem);
  uint64_t* empty_bar = reinterpret_cast<uint64_t*>(fe_smem + 128);
  T* ring = reinterpret_cast<T*>(fe_smem + 256);
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool reduce = P.reduce_op != FE_REDUCE_NONE;
  const int ni = P.n_inputs, stages = P.stages;
  const long long nchunks = P.n / CHUNK;
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], FE_THREADS / 32);
    }
    fence_mbar_init();
  }
  __syncthreads();
  pdl_launch_dependents();  // the next kernel in the stream may set itself up on SMs this grid leaves
  pdl_wait_prior_grids();   // the kernel before this one has completed: its outputs may be this one's inputs
  T acc[W];
#pragma unroll
  for (int w = 0; w < W; ++w) acc[w] = fe_identity<T>(P.reduce_op);

  if (warp == FE_THREADS / 32) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, armed = 0, armed_phase = 0;
      bool ok = true;
      const uint64_t pol = l2_policy_evict_first();  // inputs are read once: their lines should leave L2 first
      for (long long c = blockIdx.x; c < nchunks; c += gridDim.x) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, &abort_flag)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)(ni * CHUNK * sizeof(T)));
        armed |= 1u << stage;
        armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
        T* dst = ring + (size_t)stage * ni * CHUNK;
        for (int i = 0; i < ni; ++i)
          bulk_load_1d_hint(dst + (size_t)i * CHUNK, P.in[i] + c * CHUNK, CHUNK * sizeof(T), &full_bar[stage], pol);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok || abort_flag) {
        // Unwinding: give copies that were already issued a bounded time to land.
        const uint64_t t0 = globaltimer_ns();
        for (int s = 0; s < stages; ++s) {
          if (!(armed & (1u << s))) continue;
          while (!mbar_try_wait(&full_bar[s], (armed_phase >> s) & 1u)) {
            if (globaltimer_ns() - t0 > 2000000ull) break;
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- consumers
    int stage = 0;
    uint32_t phase = 0;
    for (long long c = blockIdx.x; c < nchunks; c += gridDim.x) {
      if (!mbar_wait(&full_bar[stage], phase, &abort_flag)) break;
      RingLoader<T, U> ld;
      ld.base = ring + (size_t)stage * ni * CHUNK + tid * VE;
      ld.stride = CHUNK;
      T res[W];
      fe_eval<T, W, MAXOPS>(P, ld, res);
      // Hand the stage back only after the values computed from it exist, so that neither the compiler nor the
      // hardware can have a shared-memory load of this stage (or the arithmetic that consumes it) outstanding when
      // the producer is allowed to overwrite it.
      if (reduce) {
        // Pin every result before the arrive at no cost: an empty volatile asm that takes the value as an operand
        // makes the compiler produce it first (volatile asms keep their order, and the arrive is one), and a warp
        // issues in order, so the instruction that produced it - which could only issue once its shared-memory
        // operands had returned - has issued before the arrive does. __syncwarp brings all lanes to that point.
#pragma unroll
        for (int i = 0; i < W; ++i) FeMath<T>::pin(res[i]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        fe_accumulate<T, W>(P.reduce_op, acc, res);
      } else {
        // The global stores below take every result as an operand and cannot be moved across the arrive (both are
        // memory operations): once they have issued, the loads have returned.
        T* out = P.dst + c * CHUNK + tid * VE;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          T v[VE];
#pragma unroll
          for (int k = 0; k < VE; ++k) v[k] = res[u * VE + k];
          FeMath<T>::store16_streaming(out + u * (FE_THREADS * VE), v);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);  // this warp's reads of the stage are done
      }
      if (++stage == stages) {
        stage = 0;
        phase ^= 1;
      }
    }
    fe_scalar_range<T, MAXOPS>(P, nchunks * CHUNK, (long long)blockIdx.x * FE_THREADS + tid,
                               (long long)gridDim.x * FE_THREADS, reduce, acc[0]);
  }
  if (reduce) fe_grid_reduce<T, W, MAXOPS>(P, acc);
  __syncthreads();
  if (tid == 0 && abort_flag != 0 && P.status != nullptr) atomicExch(P.status, int(ST_WAIT_TIMEOUT));
}

// Plain-load kernel for arrays that are not 16-byte aligned and for programs without inputs.
constexpr int FE_PLAIN_U = 4;  // independent elements per thread and step (8 doubles the registers and halves the occupancy: the same bytes in flight)
template <typename T, int MAXOPS>
__global__ void __launch_bounds__(FE_THREADS)
fused_elementwise_plain_kernel(const __grid_constant__ FeKernelArgs<T, MAXOPS> P) {
  constexpr int U = FE_PLAIN_U;
  pdl_launch_dependents();
  pdl_wait_prior_grids();
  const bool reduce = P.reduce_op != FE_REDUCE_NONE;
  const long long nt = (long long)gridDim.x * blockDim.x;
  const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  T acc[U];
#pragma unroll
  for (int u = 0; u < U; ++u) acc[u] = fe_identity<T>(P.reduce_op);
  for (long long base = gtid; base < P.n; base += nt * U) {
    GlobalLoader<T, U> ld;
    ld.in = P.in;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      ld.e[u] = base + (long long)u * nt;
      ld.ok[u] = ld.e[u] < P.n;
    }
    T res[U];
    fe_eval<T, U, MAXOPS>(P, ld, res);
    if (reduce) {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (!ld.ok[u]) res[u] = fe_identity<T>(P.reduce_op);
      fe_accumulate<T, U>(P.reduce_op, acc, res);
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (ld.ok[u]) P.dst[ld.e[u]] = res[u];
    }
  }
  if (reduce) fe_grid_reduce<T, U, MAXOPS>(P, acc);
}

// ------------------------------------------------------------------------------------------------ launcher
template <typename T, int MAXOPS>
static void fill_args(FeKernelArgs<T, MAXOPS>& a, const FeProgram& prog, const void* const* inputs, long long n,
                      int reduce_op, void* dst, double* result, void* reduce_scratch, int* status) {
  a.n = n;
  for (int i = 0; i < FE_MAX_INPUTS; ++i)
    a.in[i] = i < prog.n_inputs ? static_cast<const T*>(inputs[prog.input_map[i]]) : nullptr;
  a.dst = static_cast<T*>(dst);
  a.partials = static_cast<double*>(reduce_scratch);
  a.ticket = reduce_scratch
                 ? reinterpret_cast<unsigned*>(static_cast<char*>(reduce_scratch) + FE_MAX_BLOCKS * sizeof(double))
                 : nullptr;
  a.result = result;
  a.status = status;
  a.n_ops = prog.n_ops;
  a.reduce_op = reduce_op;
  a.n_inputs = prog.n_inputs;
  a.stages = 0;
  a.head = 0;
  memcpy(a.ops, prog.ops, sizeof(FeOp) * (size_t)prog.n_ops);
}

static long long clamp_blocks(long long want, long long cap) {
  if (want > cap) want = cap;
  if (want > FE_MAX_BLOCKS) want = FE_MAX_BLOCKS;
  return want < 1 ? 1 : want;
}

// Ring geometry for a program with n_inputs arrays: 16-byte vectors per thread and step (U), stages, bytes.
// The same for both element types: a chunk is FE_THREADS x U x 16 bytes per input.
struct RingGeometry {
  int u, chunk_bytes, stages, smem_bytes;
};
static RingGeometry ring_geometry(int n_inputs, int elem_bytes) {
  // Vectors per thread and step: 4 for one or two inputs (the dispatch of an op is paid once per 16 floats,
  // which matters when few bytes move per element), 2 for three or four, 1 beyond.
  RingGeometry g;
  g.u = n_inputs <= 2 ? 4 : n_inputs <= 4 ? 2 : 1;
  // 8-byte elements: two vectors per step and three CTAs per SM measured faster than four and two (5.85 against
  // 5.29 TB/s for dst = x * 2 + 1 over 64 Mi doubles).
  if (elem_bytes == 8 && g.u == 4) g.u = 2;
  g.chunk_bytes = FE_THREADS * 16 * g.u;
  const int stage_bytes = n_inputs * g.chunk_bytes;
  // Ring budget per CTA: a third of an SM's shared memory (three CTAs per SM), or half of it for the widest
  // variant, whose stages are 16 KB per input.
  g.stages = ((g.u == 4 ? 104 : 72) * 1024) / stage_bytes;
  g.stages = g.stages < 2 ? 2 : g.stages > FE_MAX_STAGES ? FE_MAX_STAGES : g.stages;
  g.smem_bytes = 256 + g.stages * stage_bytes;
  return g;
}

void describe_fused_elementwise(int n_inputs, long long n, int elem_bytes, int num_sms, int* grid, int* block,
                                int* smem_bytes) {
  if (n_inputs < 1) {  // plain-load kernel
    const long long want = (n + FE_THREADS * 4 - 1) / (FE_THREADS * 4), cap = (long long)num_sms * 8;
    *grid = (int)clamp_blocks(want, cap);
    *block = FE_THREADS;
    *smem_bytes = 0;
    return;
  }
  const RingGeometry g = ring_geometry(n_inputs > FE_MAX_INPUTS ? FE_MAX_INPUTS : n_inputs, elem_bytes);
  int per_sm = (228 * 1024) / (g.smem_bytes + 1024 + 512);  // + per-CTA reservation and static shared memory
  if (per_sm > 7) per_sm = 7;                               // 2048 threads / 288
  if (per_sm < 1) per_sm = 1;
  *grid = (int)clamp_blocks(n / (g.chunk_bytes / elem_bytes), (long long)num_sms * per_sm);
  *block = FE_THREADS + 32;
  *smem_bytes = g.smem_bytes;
}

template <typename T, int U, int MAXOPS>
static int launch_ring(const FeProgram& prog, const void* const* inputs, long long n, int reduce_op, void* dst,
                       double* result, void* reduce_scratch, int* status, int num_sms, cudaStream_t stream, int head) {
  auto kern = fused_elementwise_ring_kernel<T, U, MAXOPS>;
  SX_ENSURE_DYN_SMEM(kern, 160 * 1024);  // the largest ring is 2 stages x 16 inputs x 4 KB + barriers
  const RingGeometry geo = ring_geometry(prog.n_inputs, (int)sizeof(T));
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, FE_THREADS + 32, geo.smem_bytes) != cudaSuccess ||
      per_sm < 1)
    return set_last_error(SX_ERR_DRIVER, "occupancy query failed for the fused elementwise ring kernel");
  auto args = std::make_unique<FeKernelArgs<T, MAXOPS>>();
  fill_args(*args, prog, inputs, n, reduce_op, dst, result, reduce_scratch, status);
  args->stages = geo.stages;
  args->head = head;
  const long long nchunks = n / (geo.chunk_bytes / (int)sizeof(T));
  const long long blocks = clamp_blocks(nchunks, (long long)num_sms * per_sm);
  const cudaError_t e = launch_kernel_ex(kern, (unsigned)blocks, FE_THREADS + 32, geo.smem_bytes, stream, 1, pdl_enabled(),
                                         *args);
  if (e != cudaSuccess) return set_last_error(SX_ERR_EXEC, cudaGetErrorString(e));
  return SX_OK;
}

template <typename T, int MAXOPS>
static int launch_plain(const FeProgram& prog, const void* const* inputs, long long n, int reduce_op, void* dst,
                        double* result, void* reduce_scratch, int* status, int num_sms, cudaStream_t stream) {
  auto kern = fused_elementwise_plain_kernel<T, MAXOPS>;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, FE_THREADS, 0) != cudaSuccess || per_sm < 1)
    return set_last_error(SX_ERR_DRIVER, "occupancy query failed for the fused elementwise kernel");
  auto args = std::make_unique<FeKernelArgs<T, MAXOPS>>();
  fill_args(*args, prog, inputs, n, reduce_op, dst, result, reduce_scratch, status);
  const long long blocks = clamp_blocks((n + FE_THREADS * FE_PLAIN_U - 1) / (FE_THREADS * FE_PLAIN_U), (long long)num_sms * per_sm);
  const cudaError_t e = launch_kernel_ex(kern, (unsigned)blocks, FE_THREADS, 0, stream, 1, pdl_enabled(), *args);
  if (e != cudaSuccess) return set_last_error(SX_ERR_EXEC, cudaGetErrorString(e));
  return SX_OK;
}

template <typename T>
static int launch_typed(const FeProgram& prog, const void* const* inputs, long long n, int reduce_op, void* dst,
                        double* result, void* reduce_scratch, int* status, int num_sms, cudaStream_t stream) {
  const bool reduce = reduce_op != FE_REDUCE_NONE;
  uintptr_t bits = reduce ? 0 : reinterpret_cast<uintptr_t>(dst);
  for (int i = 0; i < prog.n_inputs; ++i) {
    const void* p = inputs ? inputs[prog.input_map[i]] : nullptr;
    if (p == nullptr) return set_last_error(SX_ERR_INVALID, "null input array");
    bits |= reinterpret_cast<uintptr_t>(p);
  }
  if (bits % sizeof(T)) return set_last_error(SX_ERR_INVALID, "arrays must be aligned to the element size");
  bool ring = bits % 16 == 0 && prog.n_inputs > 0;
  const bool small = prog.n_ops <= FE_SMALL_OPS;
  // Arrays that all start the same distance past a 16-byte boundary (slices of aligned arrays, x[1:]): the ring kernel
  // takes them from the next boundary on and computes the few elements in front of it with its scalar path.
  int head = 0;
  const void* shifted[FE_MAX_INPUTS];
  FeProgram shifted_prog;
  if (!ring && prog.n_inputs > 0 && prog.n_inputs <= FE_MAX_INPUTS) {
    const uintptr_t off = reinterpret_cast<uintptr_t>(inputs[prog.input_map[0]]) % 16;
    bool same = off != 0 && (reduce || reinterpret_cast<uintptr_t>(dst) % 16 == off);
    for (int i = 1; same && i < prog.n_inputs; ++i)
      same = reinterpret_cast<uintptr_t>(inputs[prog.input_map[i]]) % 16 == off;
    const long long h = (long long)((16 - off) / sizeof(T));
    if (same && n > h) {
      head = (int)h;
      shifted_prog = prog;
      for (int i = 0; i < prog.n_inputs; ++i) {
        shifted[i] = static_cast<const T*>(inputs[prog.input_map[i]]) + head;
        shifted_prog.input_map[i] = i;
      }
      ring = true;
    }
  }
  const FeProgram& use_prog = head ? shifted_prog : prog;
  const void* const* use_in = head ? shifted : inputs;
  void* use_dst = (head && dst) ? static_cast<void*>(static_cast<T*>(dst) + head) : dst;
  const long long use_n = n - head;
#define FE_ARGS prog, inputs, n, reduce_op, dst, result, reduce_scratch, status, num_sms, stream
  if (!ring) return small ? launch_plain<T, FE_SMALL_OPS>(FE_ARGS) : launch_plain<T, FE_MAX_OPS>(FE_ARGS);
#undef FE_ARGS
#define FE_ARGS use_prog, use_in, use_n, reduce_op, use_dst, result, reduce_scratch, status, num_sms, stream, head
  switch (ring_geometry(prog.n_inputs, (int)sizeof(T)).u) {
    case 4: return small ? launch_ring<T, 4, FE_SMALL_OPS>(FE_ARGS) : launch_ring<T, 4, FE_MAX_OPS>(FE_ARGS);
    case 2: return small ? launch_ring<T, 2, FE_SMALL_OPS>(FE_ARGS) : launch_ring<T, 2, FE_MAX_OPS>(FE_ARGS);
    default: return small ? launch_ring<T, 1, FE_SMALL_OPS>(FE_ARGS) : launch_ring<T, 1, FE_MAX_OPS>(FE_ARGS);
  }
#undef FE_ARGS
}

int launch_fused_elementwise(const FeProgram& prog, const void* const* inputs, long long n, int reduce_op, void* dst,
                             double* result, void* reduce_scratch, int* status, int num_sms, int elem_bytes,
                             cudaStream_t stream) {
  const bool reduce = reduce_op != FE_REDUCE_NONE;
  if (n <= 0) return set_last_error(SX_ERR_INVALID, "element count must be positive");
  if (reduce && (reduce_op < 0 || reduce_op > 2)) return set_last_error(SX_ERR_INVALID, "reduce_op must be 0, 1, 2 or 255");
  if (reduce && (result == nullptr || reduce_scratch == nullptr))
    return set_last_error(SX_ERR_INVALID, "null reduction output");
  if (!reduce && dst == nullptr) return set_last_error(SX_ERR_INVALID, "null dst");
  if (elem_bytes == 4)
    return launch_typed<float>(prog, inputs, n, reduce_op, dst, result, reduce_scratch, status, num_sms, stream);
  if (elem_bytes == 8)
    return launch_typed<double>(prog, inputs, n, reduce_op, dst, result, reduce_scratch, status, num_sms, stream);
  return set_last_error(SX_ERR_INVALID, "element size must be 4 or 8");
}

}  // namespace sx
