// Operand preparation for the tensor-core GEMM: HBM-bound elementwise passes.
//
//  * split_tf32: the 3xTF32 scheme represents an fp32 value x as hi + lo with hi = tf32(x) and
//    lo = tf32(x - hi); the GEMM then accumulates hi*hi + hi*lo + lo*hi in fp32 on the tensor cores.
//  * repack_16: bring 16-bit operands whose leading dimension or base address is not a multiple of
//    16 bytes into a TMA-compatible padded buffer.
#include <cuda_bf16.h>

#include "host_api.h"
#include "sm100_ptx.cuh"

namespace sx {

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// One thread produces 4 consecutive output columns of both planes (16-byte stores).
__global__ void __launch_bounds__(256)
split_tf32_kernel(const float* __restrict__ in, long long ld_in, long long batch_stride_in, float* __restrict__ out,
                  int rows, int cols, int cols_p, int batch) {
  pdl_launch_dependents();  // the GEMM that follows may set itself up while this pass drains
  pdl_wait_prior_grids();   // the source may be the output of the kernel before this one
  const int c4n = cols_p >> 2;
  const long long per_mat = (long long)rows * c4n;
  const long long total = per_mat * batch;
  const bool vec_in = (ld_in % 4 == 0) && (batch_stride_in % 4 == 0) && (reinterpret_cast<uintptr_t>(in) % 16 == 0);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i / per_mat);
    const long long rm = i - (long long)b * per_mat;
    const int r = (int)(rm / c4n);
    const int c = (int)(rm - (long long)r * c4n) * 4;
    const float* src = in + (long long)b * batch_stride_in + (long long)r * ld_in + c;
    float x[4];
    if (vec_in && c + 4 <= cols) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(src));
      x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) x[j] = (c + j < cols) ? __ldg(src + j) : 0.0f;
    }
    float hi[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      hi[j] = tf32_round(x[j]);
      lo[j] = tf32_round(x[j] - hi[j]);
    }
    float* o_hi = out + (((long long)b * 2 + 0) * rows + r) * cols_p + c;
    float* o_lo = out + (((long long)b * 2 + 1) * rows + r) * cols_p + c;
    *reinterpret_cast<float4*>(o_hi) = make_float4(hi[0], hi[1], hi[2], hi[3]);
    *reinterpret_cast<float4*>(o_lo) = make_float4(lo[0], lo[1], lo[2], lo[3]);
  }
}

// 32x32 tiles through shared memory: reads coalesced along the input's columns, writes coalesced
// along the output's (= the input's rows).
__global__ void __launch_bounds__(256)
split_tf32_transpose_kernel(const float* __restrict__ in, long long ld_in, long long batch_stride_in,
                            float* __restrict__ out, int rows, int cols, int rows_p) {
  __shared__ float tile[32][33];
  pdl_launch_dependents();
  pdl_wait_prior_grids();
  const int b = blockIdx.z;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const float* src = in + (long long)b * batch_stride_in;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty + i * 8, c = c0 + tx;
    tile[ty + i * 8][tx] = (r < rows && c < cols) ? __ldg(src + (long long)r * ld_in + c) : 0.0f;
  }
  __syncthreads();
  float* o_hi = out + ((long long)b * 2 + 0) * cols * rows_p;
  float* o_lo = out + ((long long)b * 2 + 1) * cols * rows_p;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty + i * 8, r = r0 + tx;  // output row = input column c, output column = input row r
    if (c < cols && r < rows_p) {
      const float x = tile[tx][ty + i * 8];
      const float hi = tf32_round(x);
      o_hi[(long long)c * rows_p + r] = hi;
      o_lo[(long long)c * rows_p + r] = tf32_round(x - hi);
    }
  }
}

// Element-wise fallback of the padded copy (an output pitch that is not a multiple of 8 elements; not reached from
// the library's own planning, which always pads to 8).
__global__ void __launch_bounds__(256)
repack_kernel(const uint16_t* __restrict__ in, long long ld_in, long long batch_stride_in, uint16_t* __restrict__ out,
              long long ld_out, int rows, int cols, int batch) {
  const long long per_mat = (long long)rows * ld_out;
  const long long total = per_mat * batch;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i / per_mat);
    const long long rm = i - (long long)b * per_mat;
    const int r = (int)(rm / ld_out);
    const int c = (int)(rm - (long long)r * ld_out);
    out[i] = c < cols ? in[(long long)b * batch_stride_in + (long long)r * ld_in + c] : uint16_t(0);
  }
}

// Rows of 16-bit elements whose pitch or base is not a multiple of 16 bytes -> rows of `ld_out_vec` 16-byte vectors.
// One thread per output vector: it loads the one or two aligned 16-byte granules that hold its 16 source bytes and
// shifts them into place (the byte offset inside the granule is even, 0..14), so global memory sees only aligned
// 16-byte accesses - three memory instructions per 16 bytes where an element-wise copy needs sixteen. A granule is
// only touched if at least one byte of it belongs to the row, so nothing outside the operand's 16-byte granules is
// read. Bytes past the end of a row are written as zero.
__global__ void __launch_bounds__(256)
repack_rows16_kernel(const uint8_t* __restrict__ in, long long ld_in_bytes, long long batch_stride_in_bytes,
                     uint4* __restrict__ out, long long ld_out_vec, int rows, long long row_bytes, int batch) {
  pdl_launch_dependents();
  pdl_wait_prior_grids();
  const long long per_mat = (long long)rows * ld_out_vec;
  const long long total = per_mat * batch;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i / per_mat);
    const long long rm = i - (long long)b * per_mat;
    const int r = (int)(rm / ld_out_vec);
    const long long o = (rm - (long long)r * ld_out_vec) * 16;  // byte offset inside the row
    uint32_t res[4] = {0u, 0u, 0u, 0u};
    if (o < row_bytes) {
      const uint8_t* row = in + (long long)b * batch_stride_in_bytes + (long long)r * ld_in_bytes;
      const uintptr_t addr = reinterpret_cast<uintptr_t>(row + o);
      const unsigned sh = (unsigned)(addr & 15);
      const uint4* g = reinterpret_cast<const uint4*>(addr - sh);
      const uint4 v0 = __ldg(g);
      uint4 v1 = make_uint4(0u, 0u, 0u, 0u);
      if (sh != 0 && reinterpret_cast<uintptr_t>(row + row_bytes) > reinterpret_cast<uintptr_t>(g + 1)) v1 = __ldg(g + 1);
      const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      const unsigned sw = sh >> 2, bits = (sh & 3) * 8;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (sw == (unsigned)q) {
#pragma unroll
          for (int k = 0; k < 4; ++k) res[k] = __funnelshift_r(w[q + k], w[q + k + 1], bits);
        }
      }
      const long long valid = row_bytes - o;  // source bytes that belong to this vector
      if (valid < 16) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const long long left = valid - 4 * k;
          if (left <= 0) res[k] = 0u;
          else if (left < 4) res[k] &= (1u << (8 * (int)left)) - 1u;
        }
      }
    }
    out[i] = make_uint4(res[0], res[1], res[2], res[3]);
  }
}

static int grid_for(long long work_items) {
  long long blocks = (work_items + 255) / 256;
  const long long cap = 148 * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

int launch_split_tf32(const float* in, long long ld_in, long long batch_stride_in, float* out, int rows, int cols,
                      int cols_p, int batch, cudaStream_t stream) {
  if (cols_p % 4 != 0 || cols_p < cols) return SX_ERR_INVALID;
  const long long items = (long long)rows * (cols_p / 4) * batch;
  return launch_kernel_ex(split_tf32_kernel, (unsigned)grid_for(items), 256u, 0, stream, 1, pdl_enabled(), in, ld_in,
                          batch_stride_in, out, rows, cols, cols_p, batch) == cudaSuccess
             ? SX_OK
             : SX_ERR_EXEC;
}

int launch_split_tf32_transpose(const float* in, long long ld_in, long long batch_stride_in, float* out, int rows,
                                int cols, int rows_p, int batch, cudaStream_t stream) {
  if (rows_p % 4 != 0 || rows_p < rows || batch > 65535) return SX_ERR_INVALID;
  dim3 grid((cols + 31) / 32, (rows_p + 31) / 32, batch);
  if (grid.y > 65535) return SX_ERR_INVALID;
  split_tf32_transpose_kernel<<<grid, 256, 0, stream>>>(in, ld_in, batch_stride_in, out, rows, cols, rows_p);
  return cudaGetLastError() == cudaSuccess ? SX_OK : SX_ERR_EXEC;
}

int launch_repack_16(const void* in, long long ld_in, long long batch_stride_in, void* out, long long ld_out,
                     int rows, int cols, int batch, cudaStream_t stream) {
  if (ld_out % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(in) % 2 == 0) {
    const long long vecs = (long long)rows * (ld_out / 8) * batch;
    return launch_kernel_ex(repack_rows16_kernel, (unsigned)grid_for(vecs), 256u, 0, stream, 1, pdl_enabled(),
                            static_cast<const uint8_t*>(in), ld_in * 2, batch_stride_in * 2, static_cast<uint4*>(out),
                            ld_out / 8, rows, (long long)cols * 2, batch) == cudaSuccess
               ? SX_OK
               : SX_ERR_EXEC;
  }
  const long long items = (long long)rows * ld_out * batch;
  repack_kernel<<<grid_for(items), 256, 0, stream>>>(
      static_cast<const uint16_t*>(in), ld_in, batch_stride_in, static_cast<uint16_t*>(out), ld_out, rows, cols,
      batch);
  return cudaGetLastError() == cudaSuccess ? SX_OK : SX_ERR_EXEC;
}

}  // namespace sx
