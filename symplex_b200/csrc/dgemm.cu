// Double-precision C = A.B for the f64 twins of the thin GEMM ABI (blas_dgemm / cache_tiled_dgemm_thin,
// rust-engine/src/phase3_jit.rs:449-461,676-685) that TensorMatMul traces with element type F64 call.
//
// CUDA-core kernel (the fp64 rate of a B200 is the same on and off the tensor cores): 64 x 64 output tile per CTA,
// 256 threads, 4 x 4 outputs per thread (four consecutive rows, four columns 16 apart: the 16 threads of a half-warp
// then read 16 consecutive doubles of a B row, one conflict-free shared-memory wavefront, where four consecutive
// columns per thread put the half-warp on four banks), operands staged through shared memory in k-slabs of 16 with
// register prefetch of the next slab. The arithmetic is the reference's cache_tiled_dgemm (rust-engine/src/phase3_jit.rs:
// 578-650) element for element: within each block of KC = 128 consecutive k an accumulator starts at 0 and takes
// acc = acc + a*b with the product and the sum rounded separately (Rust does not contract them), in increasing k;
// the block's accumulator is then added to C, blocks in increasing k. Neither the reference's M / N tiling nor this
// kernel's changes that order, so the two agree bit for bit.
#include "host_api.h"
#include "sm100_ptx.cuh"

namespace sx {

namespace {
constexpr int DT = 64;   // tile edge
constexpr int DK = 16;   // k-slab
constexpr int KC = 128;  // the reference's k block: one accumulator chain per block, then one add into C

__global__ void __launch_bounds__(256) dgemm_kernel(const double* __restrict__ A, long long lda,
                                                   const double* __restrict__ B, long long ldb, double* __restrict__ C,
                                                   long long ldc, int M, int N, int K) {
  __shared__ double sA[DK][DT + 1];  // [k][m]: column reads by the 4 x 4 micro-tile are conflict free
  __shared__ double sB[DK][DT];      // [k][n]
  pdl_launch_dependents();  // the next kernel in the stream may set itself up while this grid drains
  pdl_wait_prior_grids();   // the operands may be the output of the kernel before this one
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // micro-tile: rows ty*4 + i, columns tx + 16*j
  const int m0 = blockIdx.y * DT, n0 = blockIdx.x * DT;
  // loaders: A slab is 64 rows x 16 k (each thread 4 elements of one row), B slab 16 k x 64 n (4 of one k-row)
  const int a_r = tid >> 2, a_k = (tid & 3) * 4;
  const int b_k = tid >> 4, b_n = (tid & 15) * 4;
  double acc[4][4] = {};  // C so far
  double blk[4][4] = {};  // the current KC block's chain
  double ra[4], rb[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = m0 + a_r, k = k0 + a_k + i;
      ra[i] = (r < M && k < K) ? A[(long long)r * lda + k] : 0.0;
      const int kk = k0 + b_k, n = n0 + b_n + i;
      rb[i] = (kk < K && n < N) ? B[(long long)kk * ldb + n] : 0.0;
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += DK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sA[a_k + i][a_r] = ra[i];
      sB[b_k][b_n + i] = rb[i];
    }
    __syncthreads();
    if (k0 + DK < K) fetch(k0 + DK);
    const int kmax = K - k0 < DK ? K - k0 : DK;  // the chain has exactly K links: padding is never multiplied
    auto step = [&](int k) {
      double a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = sA[k][ty * 4 + i];
        b[i] = sB[k][tx + 16 * i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) blk[i][j] = __dadd_rn(blk[i][j], __dmul_rn(a[i], b[j]));
    };
    if (kmax == DK) {  // a whole slab: unrolled, so the loads of the next k run under the arithmetic of this one
#pragma unroll
      for (int k = 0; k < DK; ++k) step(k);
    } else {
      for (int k = 0; k < kmax; ++k) step(k);
    }
    if ((k0 + DK) % KC == 0 || k0 + DK >= K) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = __dadd_rn(acc[i][j], blk[i][j]);
          blk[i][j] = 0.0;
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = m0 + ty * 4 + i;
    if (r >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n < N) C[(long long)r * ldc + n] = acc[i][j];
    }
  }
}
}  // namespace

int launch_dgemm(const double* A, long long lda, const double* B, long long ldb, double* C, long long ldc, int M, int N,
                 int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return SX_ERR_INVALID;
  const dim3 grid((N + DT - 1) / DT, (M + DT - 1) / DT, 1);
  if (grid.y > 65535) return SX_ERR_INVALID;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, dgemm_kernel, A, lda, B, ldb, C, ldc, M, N, K) == cudaSuccess ? SX_OK : SX_ERR_EXEC;
}

}  // namespace sx
