// Fused epilogue shared by the GEMM kernels: one thread owns one output row and processes it in strips of
// 32 consecutive columns taken from TMEM (tcgen05.ld 32x32b.x32):
//     y = act(alpha * acc + beta * residual + bias[col])   ->  fp32 or bf16 (round to nearest even)
// written with 16-byte stores when the row is aligned, element-wise at ragged edges.
//
// The chain is the reference's fusable pattern [MatMul, Mul, Add, act] plus FUSED_GEMM's beta term
// (rust-engine/src/fusion_engine.rs:1587-1623, include/symplex/optimizer/egraph.h:74-77).
#pragma once
#include <cuda_bf16.h>

#include "gemm_params.h"

namespace sx {

__device__ __forceinline__ float tanh_mufu(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// kFast = true: every smooth activation is one MUFU tanh (rel. error ~2^-11; used by the bf16-input
// kernels, tolerance 1e-2):  sigmoid(x) = 0.5 + 0.5 tanh(x/2), silu(x) = x sigmoid(x),
// gelu(x) = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))).
// kFast = false: accurate device functions (fp32 path, tolerance 1e-5).
// The switch sits outside the element loops so each case is straight-line code over 32 independent values.
template <bool kFast>
__device__ __forceinline__ void activation32(float (&v)[32], int act) {
  switch (act) {
    case ACT_RELU:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
      break;
    case ACT_GELU:
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float x = v[j];
        if constexpr (kFast) {
          const float u = x * fmaf(0.0356774081f, x * x, 0.7978845608f);
          const float h = 0.5f * x;
          v[j] = fmaf(h, tanh_mufu(u), h);
        } else {
          const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
          v[j] = 0.5f * x * (1.0f + tanhf(u));
        }
      }
      break;
    case ACT_SIGMOID:
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if constexpr (kFast) v[j] = fmaf(0.5f, tanh_mufu(0.5f * v[j]), 0.5f);
        else v[j] = 1.0f / (1.0f + expf(-v[j]));
      }
      break;
    case ACT_TANH:
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if constexpr (kFast) v[j] = tanh_mufu(v[j]);
        else v[j] = tanhf(v[j]);
      }
      break;
    case ACT_SILU:
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if constexpr (kFast) {
          const float h = 0.5f * v[j];
          v[j] = fmaf(h, tanh_mufu(h), h);
        } else {
          v[j] = v[j] / (1.0f + expf(-v[j]));
        }
      }
      break;
    default: break;
  }
}

template <typename OutT>
struct EpilogueCtx {
  OutT* __restrict__ C;
  const OutT* __restrict__ R;
  const float* __restrict__ bias;
  float alpha, beta;
  int act, N;
  bool vec_ok, bias_vec;

  __device__ __forceinline__ explicit EpilogueCtx(const GemmParams& p)
      : C(reinterpret_cast<OutT*>(p.C)), R(reinterpret_cast<const OutT*>(p.residual)), bias(p.bias), alpha(p.alpha),
        beta(p.beta), act(p.act), N(p.N) {
    constexpr int VEC = 16 / int(sizeof(OutT));
    vec_ok = (p.ldc % VEC == 0) && (p.c_batch_stride % VEC == 0) && (reinterpret_cast<uintptr_t>(p.C) % 16 == 0);
    bias_vec = reinterpret_cast<uintptr_t>(p.bias) % 16 == 0;  // tile columns start at multiples of 32
  }

  // v: raw accumulators of columns [col0, col0 + 32) of one row, replaced by the final values
  // act(alpha v + beta R + bias). row_off: element offset of that row in C. col0 < N is required and all
  // lanes of a warp must agree on col0.
  template <bool kFast>
  __device__ __forceinline__ void math(float (&v)[32], bool row_ok, long long row_off, int col0) const {
    if (alpha != 1.0f) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= alpha;
    }
    if (R != nullptr && row_ok) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < N) v[j] += beta * float(R[row_off + col0 + j]);
    }
    if (bias != nullptr) {
      if (bias_vec && col0 + 32 <= N) {
        // all lanes read the same 128 bytes: eight broadcast 16-byte loads instead of 32 scalar ones
        const float4* b4 = reinterpret_cast<const float4*>(bias + col0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 b = __ldg(b4 + j);
          v[4 * j] += b.x; v[4 * j + 1] += b.y; v[4 * j + 2] += b.z; v[4 * j + 3] += b.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += (col0 + j < N) ? __ldg(bias + col0 + j) : 0.0f;
      }
    }
    activation32<kFast>(v, act);
  }

  // 8 consecutive values -> one 16-byte chunk of the output type (fp32: two chunks via pack4).
  static __device__ __forceinline__ uint4 pack8_bf16(const float* v) {
    __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]);
    __nv_bfloat162 h1 = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]);
    __nv_bfloat162 h3 = __floats2bfloat162_rn(v[6], v[7]);
    uint4 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&h0);
    pk.y = *reinterpret_cast<uint32_t*>(&h1);
    pk.z = *reinterpret_cast<uint32_t*>(&h2);
    pk.w = *reinterpret_cast<uint32_t*>(&h3);
    return pk;
  }

  // Final values of one strip straight to global memory.
  __device__ __forceinline__ void store(const float (&v)[32], bool row_ok, long long row_off, int col0) const {
    if (!row_ok) return;
    OutT* dst = C + row_off + col0;
    if (vec_ok && col0 + 32 <= N) {
      if constexpr (sizeof(OutT) == 4) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; j += 8) *reinterpret_cast<uint4*>(dst + j) = pack8_bf16(v + j);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < N) dst[j] = OutT(v[j]);
    }
  }

  template <bool kFast>
  __device__ __forceinline__ void strip(float (&v)[32], bool row_ok, long long row_off, int col0) const {
    math<kFast>(v, row_ok, row_off, col0);
    store(v, row_ok, row_off, col0);
  }

  // Final values of one strip into a 128-byte-swizzled staging tile of 32 rows x 128 bytes (the layout a
  // SWIZZLE_128B tensor map expects): this lane's row, 16-byte chunk c stored at chunk position c ^ (row & 7).
  // `first_chunk` is where this strip starts inside the 128-byte row (bf16: 0 or 4; fp32: 0).
  __device__ __forceinline__ void stage(const float (&v)[32], uint8_t* tile, int lane, int first_chunk) const {
    uint8_t* row = tile + lane * 128;
    const int sw = lane & 7;
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<float4*>(row + (((first_chunk + c) ^ sw) << 4)) =
            make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4*>(row + (((first_chunk + c) ^ sw) << 4)) = pack8_bf16(v + 8 * c);
    }
  }
};

}  // namespace sx
