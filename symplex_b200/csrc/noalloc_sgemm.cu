// symplex_b200_sgemm_noalloc: the fp32 (3xTF32) GEMM for callers that must not allocate.
//
// Who needs this: code that runs after a process has handed all of its GPU memory to its own allocator (a
// cudaMalloc there fails or fragments the pool), serving and control loops with a "no allocation after
// start-up" rule, and latency-sensitive callers for whom the implicit device-wide synchronisation of
// cudaMalloc / cudaFree is unacceptable. The regular fp32 entry points need scratch for the {hi, lo} tf32
// operand planes and take it from a grow-only pool (cudaMalloc on growth) or from the caller; this one keeps
// the planes in a fixed array that is part of the library image instead.
//
// Cost and limits: SYMPLEX_B200_NOALLOC_SCRATCH_BYTES (16 MiB) of device memory on every GPU that loads the
// library, held until the process exits. A problem fits if  8 * (M + N) * round_up(K, 4) + 512  bytes do.
// Every call uses the same array: two calls whose GPU work can overlap (different streams without an
// ordering between them, or different host threads) race on it - serialise them. The planes are rewritten in
// full (padding columns included) by each call before they are read, so nothing has to be cleared between
// calls and stale contents of an earlier, larger problem are never observed.
//
// Failures: the kernels' bounded waits report through a status word that is a second variable of the library image
// (below), not through the pooled entry points' word. symplex_b200_noalloc_status reads and clears it, again without
// allocating; a caller that never asks never learns that a wait ran out.
// "Calls no allocating routine" is about this code: the first CUDA call of a process on a device creates its
// context and loads the library's kernels, which is also when the 16 MiB array becomes resident.
#include <mutex>

#include "../../include/symplex_b200.h"
#include "host_api.h"

namespace sx {

// The scratch itself. In host code this name is only a handle for cudaGetSymbolAddress; the usable device
// address is looked up once per device (below) and passed to the kernels as an ordinary pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SYMPLEX_B200_NOALLOC_SCRATCH_BYTES];
static __device__ int g_noalloc_status;  // written by a kernel whose bounded wait expired

struct NoAllocDevice {
  bool ready = false;
  unsigned char* scratch = nullptr;
  int* status = nullptr;
  int num_sms = 0;
};
static NoAllocDevice g_na_dev[16];
static std::mutex g_na_mu;

// Once per device, with that device current: resolve the device addresses of the two symbols above.
static int noalloc_setup(NoAllocDevice** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return set_last_error(SX_ERR_DRIVER, "sgemm_noalloc: no current CUDA device");
  if (dev < 0 || dev >= 16) return set_last_error(SX_ERR_INVALID, "sgemm_noalloc: device ordinal out of range");
  std::lock_guard<std::mutex> lk(g_na_mu);
  NoAllocDevice& d = g_na_dev[dev];
  if (!d.ready) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10)
      return set_last_error(SX_ERR_DRIVER, "sgemm_noalloc: the current device is not an sm_100 GPU");
    if (cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return set_last_error(SX_ERR_DRIVER, "sgemm_noalloc: cannot query the SM count");
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return set_last_error(SX_ERR_DRIVER, "sgemm_noalloc: cudaGetSymbolAddress(scratch) failed");
    d.scratch = static_cast<unsigned char*>(p);
    e = cudaGetSymbolAddress(&p, g_noalloc_status);
    if (e != cudaSuccess || p == nullptr)
      return set_last_error(SX_ERR_DRIVER, "sgemm_noalloc: cudaGetSymbolAddress(status) failed");
    d.status = static_cast<int*>(p);
    d.ready = true;
  }
  *out = &d;
  return SX_OK;
}

}  // namespace sx

using namespace sx;

extern "C" int symplex_b200_sgemm_noalloc(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                                          void* stream) {
  if (M < 0 || N < 0 || K < 0) return set_last_error(SX_ERR_INVALID, "sgemm_noalloc: negative dimension");
  if (M == 0 || N == 0) return SX_OK;
  if (K == 0) return set_last_error(SX_ERR_INVALID, "sgemm_noalloc: K == 0 is not supported");
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL)
    return set_last_error(SX_ERR_INVALID, "sgemm_noalloc: dimension exceeds 2^31-1");
  if (!A || !B || !C) return set_last_error(SX_ERR_INVALID, "sgemm_noalloc: null matrix pointer");
  const long long kp = (K + 3) / 4 * 4;
  const size_t a_bytes = (size_t)2 * M * kp * 4;
  const size_t b_off = (a_bytes + 255) & ~size_t(255);
  const size_t b_bytes = (size_t)2 * N * kp * 4;
  if ((double)M * kp * 8.0 + (double)N * kp * 8.0 + 512.0 > (double)SYMPLEX_B200_NOALLOC_SCRATCH_BYTES ||
      b_off + b_bytes > (size_t)SYMPLEX_B200_NOALLOC_SCRATCH_BYTES)
    return set_last_error(SX_ERR_INVALID,
                          "sgemm_noalloc: problem needs more than the fixed 16 MiB scratch "
                          "(8*(M+N)*round_up(K,4)+512 bytes); use symplex_b200_gemm or symplex_b200_gemm_ws");
  NoAllocDevice* d = nullptr;
  int rc = noalloc_setup(&d);
  if (rc != SX_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* Ap = reinterpret_cast<float*>(d->scratch);
  float* Bp = reinterpret_cast<float*>(d->scratch + b_off);
  rc = launch_split_tf32(A, K, M * K, Ap, (int)M, (int)K, (int)kp, 1, s);
  if (rc != SX_OK) return set_last_error(rc, "sgemm_noalloc: operand split (A) launch failed");
  rc = launch_split_tf32_transpose(B, N, K * N, Bp, (int)K, (int)N, (int)kp, 1, s);
  if (rc != SX_OK) return set_last_error(rc, "sgemm_noalloc: operand split (B) launch failed");
  TcGemmArgs g{};
  g.M = M; g.N = N; g.K = K;
  g.batch = 1;
  g.out_bf16 = 0;
  g.A = Ap; g.lda = kp; g.a_plane_stride = M * kp;
  g.B = Bp; g.ldb = kp; g.b_plane_stride = N * kp;
  g.C = C; g.ldc = N; g.c_batch_stride = M * N;
  g.alpha = 1.0f; g.beta = 0.0f; g.act = 0;
  g.status = d->status;
  g.num_sms = d->num_sms;
  // same tile rule as the pooled fp32 path, so both entry points run the identical kernel configuration
  g.bn = (N > 64 && ((M + 127) / 128) * ((N + 127) / 128) >= d->num_sms) ? 128 : 64;
  rc = launch_gemm_tf32x3(g, s);
  if (rc != SX_OK) return set_last_error(rc, "sgemm_noalloc: GEMM kernel launch failed");
  return SX_OK;
}

extern "C" int symplex_b200_noalloc_status(void* stream) {
  NoAllocDevice* d = nullptr;
  int rc = noalloc_setup(&d);
  if (rc != SX_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int status = 0;  // a pageable stack word: the copy is staged by the driver, nothing is allocated here
  if (cudaMemcpyAsync(&status, d->status, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess) {
    cudaGetLastError();
    return set_last_error(SX_ERR_EXEC, "noalloc_status: reading the status word failed");
  }
  if (status == 0) return SX_OK;
  if (cudaMemsetAsync(d->status, 0, sizeof(int), s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) {
    cudaGetLastError();
    return set_last_error(SX_ERR_EXEC, "noalloc_status: clearing the status word failed");
  }
  return set_last_error(SX_ERR_TIMEOUT, "sgemm_noalloc: a device-side wait timed out; the output is not valid");
}
