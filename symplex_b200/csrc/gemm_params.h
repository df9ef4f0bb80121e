// Parameter block shared by the tcgen05 GEMM kernels and their host launchers.
#pragma once
#include <stdint.h>

namespace sx {

enum Activation : int {
  ACT_NONE = 0,
  ACT_RELU = 1,
  ACT_GELU = 2,  // tanh form: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
  ACT_SIGMOID = 3,
  ACT_TANH = 4,
  ACT_SILU = 5,
};

enum KernelStatus : int {
  ST_OK = 0,
  ST_WAIT_TIMEOUT = 5,  // a bounded mbarrier wait ran out; the kernel unwound and returned
};

// One launch computes, for every z in [0, batch):
//   C_z = act(alpha * sum_s A[z*a_planes + a_plane[s]] . B[z*b_planes + b_plane[s]] + beta * R_z + bias)
// nseg = 1 is a plain GEMM; nseg = 3 with planes (hi,hi), (hi,lo), (lo,hi) is the 3xTF32 product.
struct GemmParams {
  int M, N, K;
  int batch;
  int nseg;
  int a_plane[3];
  int b_plane[3];
  int a_planes, b_planes;
  void* C;
  long long ldc;             // elements
  long long c_batch_stride;  // elements
  const float* bias;         // fp32[N], broadcast over rows; may be null
  const void* residual;      // same dtype/layout as C; may be null (beta ignored then)
  float alpha, beta;
  int act;
  int* status;  // device word, receives KernelStatus on failure
  int m_tiles, n_tiles, group_m;
  int n_dst;  // 0: epilogue stores straight from registers; >= 1: staged in shared memory and written by TMA
              // to n_dst destinations (the local C first, then the same tile of every peer GPU's C)
  // shared-memory descriptor fields for a B tile held MN-major (row-major B[K,N])
  uint32_t b_lbo, b_sbo, b_kstep;
};

// Tensor maps of the output destinations of the TMA-store epilogue (local C, then peers' C).
constexpr int MAX_DST = 8;

}  // namespace sx
