// Internal host-side interfaces between the launchers (one per .cu file) and the C-ABI layer.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>

// Raise a kernel's dynamic shared-memory limit once per device. The static lives at the expansion site, i.e.
// once per template instantiation of the launcher that uses it.
#define SX_ENSURE_DYN_SMEM(kern, bytes)                                                                        \
  do {                                                                                                         \
    static std::atomic<uint32_t> done__{0};                                                                    \
    int dev__ = 0;                                                                                             \
    cudaGetDevice(&dev__);                                                                                     \
    if (dev__ < 0 || dev__ >= 32 || !((done__.load(std::memory_order_relaxed) >> dev__) & 1u)) {                \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)       \
        return sx::set_last_error(-1, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed for " #kern);   \
      if (dev__ >= 0 && dev__ < 32) done__.fetch_or(1u << dev__);                                              \
    }                                                                                                          \
  } while (0)

namespace sx {

// One launch path for the tcgen05 kernels: an optional cluster of `cluster_x` CTAs and, with `pdl`, the
// programmatic-stream-serialization attribute (the kernel may start its set-up while the kernel before it in the
// stream is draining; it waits for that kernel inside, see pdl_wait_prior_grids in sm100_ptx.cuh).
template <typename Kern, typename... Args>
inline cudaError_t launch_kernel_ex(Kern kern, unsigned grid, unsigned block, size_t dyn_smem, cudaStream_t stream,
                                    unsigned cluster_x, bool pdl, const Args&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.dynamicSmemBytes = dyn_smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}
bool pdl_enabled();  // the "pdl" option (capi.cu)


// Status codes returned through the C ABI. They mirror the failure classes of the reference's
// CudaError enum (rust-engine/src/cuda_backend.rs:35-50); TIMEOUT has no counterpart there.
enum : int {
  SX_OK = 0,
  SX_ERR_DRIVER = -1,   // DriverError / NoGpuFound
  SX_ERR_INVALID = -2,  // InvalidParam
  SX_ERR_OOM = -3,      // OutOfMemory
  SX_ERR_EXEC = -4,     // ExecutionError
  SX_ERR_TIMEOUT = -5,  // a bounded device-side wait expired
};

// Arguments of one tensor-core GEMM launch on device-resident, TMA-compatible operands
// (16-byte aligned base pointers, leading dimensions that are multiples of 16 bytes).
struct TcGemmArgs {
  int kind;      // 0: bf16 inputs (kind::f16), 1: fp32 containers read as tf32 (kind::tf32)
  int out_bf16;  // output dtype: 0 fp32, 1 bf16
  int b_mn;      // 1: B is row-major [K,N] (N contiguous); 0: B is [N,K] (K contiguous)
  int bn;        // tile width: 256, 128 or 64
  long long M, N, K;
  int batch;
  int nseg;
  int a_plane[3], b_plane[3];
  int a_planes, b_planes;  // planes per batch entry
  int za, zb;              // total planes in the A / B allocations (batch * planes)
  const void* A;
  long long lda, a_plane_stride;  // elements
  const void* B;
  long long ldb, b_plane_stride;
  void* C;
  long long ldc, c_batch_stride;
  const float* bias;
  const void* residual;
  float alpha, beta;
  int act;
  int* status;
  int num_sms;
  int group_m;
  int tma_store;               // pair kernels: stage the output in shared memory and write it with TMA
  int n_peers;                 // pair kernels: also write every tile to the same offset of these buffers
  const void* peer_C[7];       //   (other GPUs' copies of C, mapped into this process)
  // Exchange mode (Exchange in gemm_params.h; 0 with n_peers > 0 means XCHG_EPILOGUE_TMA). The forwarder modes
  // order the ranks inside the kernel and need the flag blocks, the call number and this GPU's counter word.
  int xchg;
  int my_rank, peer_rank[7];
  void* mc_C;
  int* flags;
  int* peer_flags[7];
  int epoch;
  unsigned* xchg_counter;
  unsigned long long wait_limit_ns;  // 0 = the default bound (2 s)
  int fault_stop_early;              // single-CTA kernel, self-test only
  // 512 x 256 pair kernel: stream-K over the k-blocks of all tiles (GemmParams::sk_*). Not with peers.
  float* sk_ws;
  int* sk_flags;
  int sk_epoch;
};
// Stream-K of the 512 x 256 pair kernel: bytes of partial-sum workspace and flag words for a device with num_sms SMs.
size_t stream_k_workspace_bytes(int num_sms);
int stream_k_flag_words(int num_sms);
int stream_k_work_items(int pair, int pairs, int tiles, int nkb, int* out, int cap);
int stream_k_contributors(int pair, int pairs, int tiles, int nkb, int tile);

int launch_gemm_tc(const TcGemmArgs& a, cudaStream_t stream);
int pick_bn(long long M, long long N, int batch, int num_sms, int forced);
// bf16 GEMM on CTA pairs (256x256 tiles, tcgen05 cta_group::2); operand conventions of launch_gemm_tc, a.bn ignored.
int launch_gemm_pair(const TcGemmArgs& a, cudaStream_t stream);
// 3xTF32 GEMM on pre-split operands: A planes [batch][2][M][lda], B planes [batch][2][N][ldb], both K contiguous;
// a.bn is 128 or 64. Fields kind / b_mn / nseg / *_plane* of TcGemmArgs are ignored.
int launch_gemm_tf32x3(const TcGemmArgs& a, cudaStream_t stream);

// Records `msg` as the calling thread's last error and returns `code`.
int set_last_error(int code, const char* msg);

// fp32 GEMM with the tf32 hi/lo split done in shared memory (no pre-pass, no scratch): raw fp32 operands,
// 128 x 64 tiles. For small and batched problems; operands must satisfy f32_fused_operands_ok.
int launch_gemm_f32_fused(const TcGemmArgs& a, cudaStream_t stream);
bool f32_fused_operands_ok(const TcGemmArgs& a);
// CTAs per output tile (1, 2 or 4; > 1 = split-K over a thread-block cluster) for `tiles` tiles of 128 x 64.
int f32_fused_split_k(long long tiles, long long K, int num_sms);
// The same arithmetic for problems with at most 64 rows (batches of tiny products): 64 x 64 tiles (M = 64 MMA
// shape) and separate rings for raw and converted tiles (gemm_f32_small_sm100.cu).
int launch_gemm_f32_small(const TcGemmArgs& a, cudaStream_t stream);
// Rows of one problem's output tile: 64 (problems with at most 64 rows go to launch_gemm_f32_small), else 128.
int f32_fused_tile_rows(long long M);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda dependency).
int encode_tensor_map_3d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, const uint64_t dims[3],
                         const uint64_t strides_bytes[2], const uint32_t box[3], bool swizzle128 = true);

// Operand preparation kernels (prep_kernels.cu).
// fp32 [batch][rows][cols] (leading dimension ld_in) -> planes [batch][2][rows][cols_p]:
// plane 0 = tf32-rounded value, plane 1 = tf32-rounded remainder; columns >= cols are zero.
int launch_split_tf32(const float* in, long long ld_in, long long batch_stride_in, float* out, int rows, int cols,
                      int cols_p, int batch, cudaStream_t stream);
// Same split for a matrix that is stored transposed relative to what the GEMM wants:
// fp32 [batch][rows][cols] -> planes [batch][2][cols][rows_p] (out[c][r] = in[r][c]); rows >= rows are zero.
int launch_split_tf32_transpose(const float* in, long long ld_in, long long batch_stride_in, float* out, int rows,
                                int cols, int rows_p, int batch, cudaStream_t stream);
// Copy a 2-byte-element matrix into a buffer whose leading dimension is ld_out (zero padded).
int launch_repack_16(const void* in, long long ld_in, long long batch_stride_in, void* out, long long ld_out,
                     int rows, int cols, int batch, cudaStream_t stream);

// Double-precision C = A.B in the reference's cache_tiled_dgemm summation order (dgemm.cu). Leading dimensions in elements.
int launch_dgemm(const double* A, long long lda, const double* B, long long ldb, double* C, long long ldc, int M, int N,
                 int K, cudaStream_t stream);

// Static shape of one GEMM kernel variant, for the planning queries of the C ABI (no GPU needed).
struct KernelShape {
  const char* name;
  int tile_m, tile_n, tile_k;  // output tile per CTA (per CTA pair when cluster == 2) and K per pipeline stage
  int mma_m, mma_n, mma_k;     // one tcgen05.mma instruction
  int threads, cluster, stages, smem_bytes, tmem_cols;
};
KernelShape describe_gemm_tc(int bn);      // gemm_sm100.cu: bf16, one CTA per tile
KernelShape describe_gemm_pair(int kmb);   // gemm_pair_sm100.cu: bf16, CTA pair, kmb = 1 (256x256) or 2 (512x256)
KernelShape describe_gemm_tf32x3(int bn);  // gemm_tf32x3_sm100.cu: fp32 from pre-split planes
KernelShape describe_gemm_f32_fused(int split_k);
KernelShape describe_gemm_f32_small();     // gemm_f32_small_sm100.cu: fp32, at most 64 rows  // gemm_f32_fused_sm100.cu: fp32, hi/lo split in shared memory

// ---- fused elementwise programs (fused_elementwise.cu) -------------------------------------------------------
// One op of a compiled program. Operand kinds: input array (value = compacted input index), immediate
// (value = the float's bits), slot (value = index into the per-thread slot file) or the previous op's result.
enum : uint8_t { FE_IN = 0, FE_IMM = 1, FE_SLOT = 2, FE_LAST = 3 };
constexpr int FE_MAX_INPUTS = 16;
constexpr int FE_MAX_SLOTS = 16;
constexpr int FE_SMALL_OPS = 64;
constexpr int FE_MAX_OPS = 1024;
constexpr int FE_MAX_BLOCKS = 2048;        // upper bound of the grid, sizes the reduction scratch
constexpr uint8_t FE_NO_DST = 0xff;
constexpr int FE_REDUCE_NONE = 255;
struct FeOp {
  uint8_t opcode, lkind, rkind, dst;  // dst: slot that receives the result, or FE_NO_DST
  uint32_t pad_;
  uint64_t l, r;                      // index, or the immediate's bits (a float's in the low word)
};
struct FeProgram {
  int n_ops = 0, n_inputs = 0, n_slots = 0;
  int input_map[FE_MAX_INPUTS];  // compacted index -> index in the caller's input list
  FeOp ops[FE_MAX_OPS];
};
struct FeSrcOp {  // layout of the reference's #[repr(C)] FusedOpDesc
  uint8_t op, lhs_src;
  uint16_t lhs_idx;
  uint8_t rhs_src, pad_;
  uint16_t rhs_idx;
};
// Resolve constants, compact the inputs that are used, and assign slots by liveness. Pure host code.
// `constants` holds n_constants values of elem_bytes (4: float, 8: double) each.
int compile_fused_program(const FeSrcOp* ops, size_t n_ops, size_t n_inputs, const void* constants,
                          size_t n_constants, int elem_bytes, FeProgram* out);
// Launch geometry the kernels use for a program with n_inputs arrays of n elements (host only; the launch
// path asks the occupancy calculator for the CTAs per SM, this uses the shared-memory arithmetic).
void describe_fused_elementwise(int n_inputs, long long n, int elem_bytes, int num_sms, int* grid, int* block,
                                int* smem_bytes);
// Device scratch of one reduction: FE_MAX_BLOCKS doubles followed by a ticket word (zero between launches).
constexpr size_t FE_REDUCE_SCRATCH_BYTES = FE_MAX_BLOCKS * sizeof(double) + 256;
// Evaluate the program over n elements of elem_bytes (4 or 8) each. inputs[] follow the caller's numbering. reduce_op 255: store to dst;
// 0 / 1 / 2: sum / max / min of the final value into *result (a device double), nothing stored to dst.
// status: device word that receives ST_WAIT_TIMEOUT if a bounded wait inside the kernel runs out.
int launch_fused_elementwise(const FeProgram& prog, const void* const* inputs, long long n, int reduce_op, void* dst,
                             double* result, void* reduce_scratch, int* status, int num_sms, int elem_bytes,
                             cudaStream_t stream);

}  // namespace sx
