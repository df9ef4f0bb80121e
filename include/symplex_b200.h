/*
 * symplex_b200 — C ABI of the B200 (sm_100a) dense-matmul kernel library.
 *
 * Everything SympleX's host code (Rust `extern "C"`, pyo3, ctypes, C++) needs in order to run its
 * tiled dense matmul and the elementwise epilogues fused into it on a B200. Plain pointers and sizes
 * only. Unless a function says otherwise it returns 0 on success or one of the negative
 * SYMPLEX_ERR_* codes; nothing throws across this boundary and there is no CPU fallback: without a
 * usable GPU every compute entry point fails with SYMPLEX_ERR_DRIVER (void entry points leave C
 * untouched and record the error for symplex_b200_last_error()).
 */
#ifndef SYMPLEX_B200_H
#define SYMPLEX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with hidden visibility; these are its exports */
#endif

/* Failure classes; same split as the reference's CudaError enum
 * (rust-engine/src/cuda_backend.rs:35-50). TIMEOUT is new: a bounded device-side wait expired. */
#define SYMPLEX_OK 0
#define SYMPLEX_ERR_DRIVER (-1)
#define SYMPLEX_ERR_INVALID (-2)
#define SYMPLEX_ERR_OOM (-3)
#define SYMPLEX_ERR_EXEC (-4)
#define SYMPLEX_ERR_TIMEOUT (-5)

/* Element types: values of the reference's ScalarType (rust-engine/src/types.rs:110-116). */
#define SYMPLEX_DT_F32 9
#define SYMPLEX_DT_BF16 11

/* Matrix layouts: values of the reference's MatrixLayout (rust-engine/src/types.rs:177-181). */
#define SYMPLEX_ROW_MAJOR 0
#define SYMPLEX_COL_MAJOR 1

/* Activations that fold into the matmul: the set accepted by is_activation /
 * matches_matmul_bias_activation (rust-engine/src/fusion_engine.rs:261-266,1587-1623). */
#define SYMPLEX_ACT_NONE 0
#define SYMPLEX_ACT_RELU 1
#define SYMPLEX_ACT_GELU 2 /* tanh form, python/symplex/_array.py:359-360 */
#define SYMPLEX_ACT_SIGMOID 3
#define SYMPLEX_ACT_TANH 4
#define SYMPLEX_ACT_SILU 5

/*
 * One (optionally strided-batched) GEMM with a fused epilogue:
 *     C = act(alpha * A.B + beta * R + bias)        A:[M,K] row-major, C,R:[M,N] row-major
 * in_dtype F32 computes on tensor cores with the 3xTF32 split (fp32-level accuracy); BF16 multiplies
 * bf16 inputs with fp32 accumulation. bias is fp32[N] broadcast over rows, or NULL. Leading
 * dimensions / batch strides are in elements; 0 selects the packed default.
 * Covers the fused chains of the reference's fusion vocabulary: [MatMul,Add], [MatMul,act],
 * [MatMul,Add,act], [MatMul,Mul,Add,act] and FUSED_GEMM = alpha.A.B + beta.C
 * (rust-engine/src/fusion_engine.rs:1587-1623, include/symplex/optimizer/egraph.h:74-77).
 */
typedef struct symplex_gemm_desc {
  int64_t M, N, K;
  int32_t batch;      /* number of independent problems, >= 1 */
  int32_t in_dtype;   /* SYMPLEX_DT_F32 or SYMPLEX_DT_BF16 (A and B) */
  int32_t out_dtype;  /* SYMPLEX_DT_F32 or SYMPLEX_DT_BF16 (C and R) */
  int32_t b_layout;   /* SYMPLEX_ROW_MAJOR: B is [K,N]; SYMPLEX_COL_MAJOR: B is stored as [N,K] */
  int64_t lda, ldb, ldc;
  int64_t a_batch_stride, b_batch_stride, c_batch_stride;
  float alpha, beta;
  int32_t activation; /* SYMPLEX_ACT_* */
  int32_t tile_n;     /* advisory tile hint like the reference's tile_m/n/k keys: 0 = auto, 64/128/256 */
} symplex_gemm_desc;

/* Fill a descriptor with defaults (batch 1, row-major B, alpha 1, beta 0, no activation). */
void symplex_b200_gemm_desc_init(symplex_gemm_desc* d, int64_t M, int64_t N, int64_t K, int32_t in_dtype,
                                 int32_t out_dtype);

/* ---- device-pointer entry points (new; the reference has no device-resident API) ------------- */

/* Bytes of scratch the GEMM described by `d` needs (operand planes for the fp32 path, padded copies
 * of operands that are not 16-byte aligned; 0 if none). */
size_t symplex_b200_gemm_workspace_bytes(const symplex_gemm_desc* d);

/* Asynchronous GEMM on `stream` (a cudaStream_t, NULL = default stream) with device pointers.
 * Scratch comes from a grow-only per-device pool owned by the library. `residual` may be NULL. */
int symplex_b200_gemm(const symplex_gemm_desc* d, const void* A, const void* B, void* C, const float* bias,
                      const void* residual, void* stream);

/* symplex_b200_gemm that additionally writes every tile of C, from inside the GEMM kernel, to the same offset of
 * `n_peers` (<= 7) other buffers: the C of other GPUs of the box, mapped into this process (CUDA IPC / symmetric
 * memory), written over NVLink by TMA stores issued from the epilogue. This is the all-gather of a row-sharded
 * product fused into the GEMM - no separate collective. bf16 inputs; C and every peer buffer need 16-byte
 * aligned rows. The caller orders the GPUs (all ranks done before C is read, and before the next call overwrites
 * it). The reference only has a planner that emits collective calls as text
 * (include/symplex/distributed/nccl_bridge.h:91-98); this is the executed counterpart. */
int symplex_b200_gemm_peers(const symplex_gemm_desc* d, const void* A, const void* B, void* C, const float* bias,
                            const void* residual, const void* const* peer_C, int32_t n_peers, void* stream);

/* Same, with caller-provided scratch of at least symplex_b200_gemm_workspace_bytes(d) bytes
 * (256-byte aligned device memory); never allocates. */
int symplex_b200_gemm_ws(const symplex_gemm_desc* d, const void* A, const void* B, void* C, const float* bias,
                         const void* residual, void* workspace, size_t workspace_bytes, void* stream);

/* Allocation-free fp32 GEMM, C = A.B (row-major, device pointers, asynchronous on `stream`). No counterpart
 * in the reference: it exists for callers that cannot allocate GPU memory at the time of the call - processes
 * whose own allocator already owns all device memory, serving loops with a no-allocation-after-start-up rule,
 * callers that cannot tolerate the device-wide synchronisation of cudaMalloc/cudaFree. The operand planes of
 * the 3xTF32 scheme live in a fixed SYMPLEX_B200_NOALLOC_SCRATCH_BYTES array inside the library (resident on
 * every GPU that loads it, until exit); this function calls no allocating routine.
 * Limit: 8*(M+N)*round_up(K,4) + 512 <= SYMPLEX_B200_NOALLOC_SCRATCH_BYTES (e.g. 1024^3 is too big by 512 B,
 * 1024 x 1024 x 1020 fits), else SYMPLEX_ERR_INVALID.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress); make that call
 * before starting any stream capture. All calls share the one array: calls whose GPU work may overlap race
 * on it and must be serialised by the caller. Nothing needs clearing between calls. */
#define SYMPLEX_B200_NOALLOC_SCRATCH_BYTES (16 * 1024 * 1024)
int symplex_b200_sgemm_noalloc(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                               void* stream);

/* Synchronise `stream` and return the device-side status of the launches since the last call:
 * 0, SYMPLEX_ERR_TIMEOUT or SYMPLEX_ERR_EXEC. */
int symplex_b200_sync_status(void* stream);

/* Message for the most recent failure on the calling thread (static storage; never NULL). */
const char* symplex_b200_last_error(void);

/* ---- host-pointer drop-ins ------------------------------------------------------------------- */

/* General form of the reference's cuda_matmul (rust-engine/src/cuda_backend.rs:1344-1385): host
 * buffers in, host buffer out, copies inside. Device buffers are cached per thread; nothing is
 * re-compiled per call. */
int symplex_b200_gemm_host(const symplex_gemm_desc* d, const void* A, const void* B, void* C, const float* bias,
                           const void* residual);

/* _symplex_core.cuda_matmul / symplex_engine.cuda_matmul_raw (python/src/lib.rs:1836-1849,
 * rust-engine/src/lib.rs:1589-1592): fp32 row-major host matrices, returns 0 or -1. */
int64_t symplex_cuda_matmul(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k);

/* _symplex_core.parallel_matmul / jit_parallel_matmul (python/src/lib.rs:1029-1062) and the Rust
 * functions behind them (rust-engine/src/x86_emitter.rs:1877-1919): same contract, returns 0
 * (also for a zero dimension, which is a no-op) or a negative SYMPLEX_ERR_* code. */
int64_t symplex_parallel_matmul(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k);
int64_t symplex_jit_parallel_matmul(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k);

/* The JIT kernel ABI of exec_matmul (rust-engine/src/x86_emitter.rs:70-77): returns 0. */
int64_t symplex_exec_matmul(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k);

/* The 7-argument fused kernel ABI of exec_fused_matmul_bias_relu
 * (rust-engine/src/x86_emitter.rs:90-100,634-770): C = max(A.B + bias[N], 0). */
int64_t symplex_exec_fused_matmul_bias_relu(const float* a, const float* b, float* c, int64_t m, int64_t n,
                                            int64_t k, const float* bias);

/* libsymplex_kernels.so entry points (kernels/matmul.c:7-18,82-101): C is fully overwritten. */
void symplex_matmul_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K);
void symplex_matmul_tiled_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K);

/* The thin GEMM ABI that JIT-compiled TensorMatMul traces call
 * (rust-engine/src/phase3_jit.rs:431-445,660-669): alpha 1, beta 0, natural leading dimensions. */
void blas_sgemm(const float* a, const float* b, float* c, size_t m, size_t n, size_t k);
void cache_tiled_sgemm_thin(const float* a, const float* b, float* c, size_t m, size_t n, size_t k);

/* Execute one serialized Instr::TensorMatMul record (rust-engine/src/types.rs:407-417,646-657,884-904: opcode
 * 0xA2, dst/lhs/rhs slot u16, m/n/k u64, element_ty, lhs_layout, rhs_layout; 34 bytes little endian) against an
 * array of host pointers indexed by slot - what the reference's JIT lowers to a blas_sgemm call
 * (rust-engine/src/phase3_jit.rs:13024-13118). Unlike the reference, which parses the layout bytes and then
 * ignores them, rhs_layout is honoured (RowMajor: [K,N]; ColMajor: stored [N,K]); F32 and BF16 element types;
 * lhs must be RowMajor. Returns 0 or a negative SYMPLEX_ERR_* code. */
int64_t symplex_b200_exec_tensor_matmul(const uint8_t* record, size_t record_len, void* const* slots, size_t nslots);

/* ---- jit::ORCJIT::execute(name, KernelArgs&) ------------------------------------------------ */

/* Same members, order and types as jit::KernelArgs (include/symplex/jit/orc_jit.h:103-114), so a C++ caller
 * passes its KernelArgs object as is. */
typedef struct symplex_kernel_args {
  void* data;           /* output tensor (host) */
  int64_t data_size;    /* bytes */
  void** input_ptrs;    /* input tensors (host) */
  int64_t num_inputs;
  int64_t* input_sizes; /* bytes each; may be NULL (then sizes are not checked) */
  int64_t M, N, K;
  int64_t batch;
} symplex_kernel_args;

/* ORCJIT::execute(kernel_name, args) (include/symplex/jit/orc_jit.h:179) for the kernels of this path, fp32,
 * row-major, host pointers: "matmul" (inputs A [batch][M][K], B [batch][K][N] -> data [batch][M][N]) and
 * "fused_matmul_bias_relu" (third input bias[N]). Names are matched on these substrings, so the reference's
 * generated names ("symplex_matmul_128x128x64", ...) work. Returns 0, or a negative SYMPLEX_ERR_* code: unknown
 * kernel, too few inputs, or a buffer smaller than the dimensions require are SYMPLEX_ERR_INVALID. */
int symplex_b200_execute(const char* kernel_name, const symplex_kernel_args* args);

/* ---- device queries -------------------------------------------------------------------------- */

/* CudaRuntime::is_available / _symplex_core.cuda_available (rust-engine/src/cuda_backend.rs:1078-1100,
 * python/src/lib.rs:1715): 1 if device 0 exists and is an sm_100 part, else 0. */
int symplex_cuda_available(void);

/* Fields of _symplex_core.cuda_device_info (python/src/lib.rs:1721-1753). */
typedef struct symplex_device_info {
  char name[256];
  int32_t compute_capability_major, compute_capability_minor;
  uint64_t total_memory_bytes;
  int32_t num_sms;
  int32_t num_cuda_cores;
  int32_t warp_size;
  int32_t max_threads_per_block;
  int32_t max_shared_memory_per_block;
  int32_t clock_mhz;
} symplex_device_info;
int symplex_cuda_device_info(symplex_device_info* out);

/* sizeof() of the structs of this header as the library was compiled: {symplex_gemm_desc, symplex_device_info,
 * symplex_fused_op, symplex_b200_target, symplex_gemm_plan}. Lets a binding written in another language check
 * its own struct definitions at load time. */
void symplex_b200_abi_sizes(int32_t out[5]);

/* Kernels launched by this library on the calling process since load (all threads). */
uint64_t symplex_b200_launch_count(void);

/* ---- fused elementwise programs (optional reduction) ------------------------------------------ */

/* FusedOpDesc of the reference, #[repr(C)], 8 bytes (rust-engine/src/x86_emitter.rs:1937-1953).
 * op: 0 add, 1 sub, 2 mul, 3 div, 4 min, 5 max, 6 neg, 7 abs, 8 sqrt, 9 exp, 10 log, 11 sin, 12 cos, 13 tanh,
 * 14 sigmoid, 15 relu (6..15 unary: rhs ignored; other codes pass lhs through).
 * lhs_src / rhs_src: 0 input array, 1 constant, 2 result of an earlier op; *_idx indexes that source.
 * As in the reference, an input or constant index out of range reads as 0; so does a reference to an op
 * that has not run yet. */
typedef struct symplex_fused_op {
  uint8_t op;
  uint8_t lhs_src;
  uint16_t lhs_idx;
  uint8_t rhs_src;
  uint8_t reserved;
  uint16_t rhs_idx;
} symplex_fused_op;

#define SYMPLEX_REDUCE_SUM 0
#define SYMPLEX_REDUCE_MAX 1
#define SYMPLEX_REDUCE_MIN 2
#define SYMPLEX_REDUCE_NONE 255

/* x86_emitter::simd_fused_elementwise_f32 / _symplex_core.simd_fused_elementwise_f32
 * (rust-engine/src/x86_emitter.rs:2442-2470, python/src/lib.rs:1686-1695): evaluate the op chain over n
 * elements of HOST arrays in one pass. reduce_op 255: the last op's values are written to dst_ptr and 0.0 is
 * returned; 0 / 1 / 2: their sum / max / min is returned and dst_ptr is not touched. n == 0 or an empty chain
 * returns 0.0. There is no error channel in the reference; on failure this returns NaN and
 * symplex_b200_last_error() says why. Limits: 1024 ops, 16 distinct input arrays, 16 values alive at once.
 * Difference from the reference, on purpose: for max / min with n not a multiple of 8 the reference ADDS the
 * maximum of the vector part and the maximum of the scalar tail (x86_emitter.rs:2347); this returns the
 * true maximum / minimum. */
double symplex_simd_fused_elementwise_f32(const symplex_fused_op* ops, size_t n_ops, const float* const* input_ptrs,
                                          size_t n_inputs, const float* constants, size_t n_constants, size_t n,
                                          uint8_t reduce_op, float* dst_ptr);

/* The f64 twin (rust-engine/src/x86_emitter.rs:2799-2828, python/src/lib.rs:1700-1709): same chain encoding on
 * double arrays and double constants; this is what the reference's Python layer calls for float64 NumPy data. */
double symplex_simd_fused_elementwise_f64(const symplex_fused_op* ops, size_t n_ops, const double* const* input_ptrs,
                                          size_t n_inputs, const double* constants, size_t n_constants, size_t n,
                                          uint8_t reduce_op, double* dst_ptr);

/* Same computation on DEVICE arrays, asynchronous on `stream`. `result` (device double, 8-byte aligned)
 * receives the reduced value when reduce_op != 255; `dst` receives the values otherwise and may alias an
 * input. Arrays that are all 16-byte aligned take the bulk-copy kernel, others a plain-load kernel.
 * No counterpart in the reference (its GPU path copies host arrays per call, cuda_backend.rs:1420-1455). */
int symplex_b200_fused_elementwise_f32(const symplex_fused_op* ops, size_t n_ops, const float* const* inputs,
                                       size_t n_inputs, const float* constants, size_t n_constants, int64_t n,
                                       int reduce_op, float* dst, double* result, void* stream);
int symplex_b200_fused_elementwise_f64(const symplex_fused_op* ops, size_t n_ops, const double* const* inputs,
                                       size_t n_inputs, const double* constants, size_t n_constants, int64_t n,
                                       int reduce_op, double* dst, double* result, void* stream);

/* cuda_backend::cuda_elementwise / symplex_engine.cuda_elementwise_raw (rust-engine/src/cuda_backend.rs:1420-1455,
 * rust-engine/src/lib.rs:1597-1626): dst[i] = a[i] <op> b[i] on host arrays, op 0 add, 1 sub, 2 mul, 3 div,
 * 4 min, 5 max. Returns 0, -1 on a CUDA error, -2 for an unknown op. */
int64_t symplex_cuda_elementwise(const float* a, const float* b, float* dst, int64_t n, int op);

/* Host-only: compile a chain and report how many slots of the per-thread slot file it needs and how many
 * distinct input arrays it reads. Returns SYMPLEX_ERR_INVALID for chains outside the limits above.
 * Needs no GPU. */
int symplex_b200_fused_program_info(const symplex_fused_op* ops, size_t n_ops, size_t n_inputs, int* n_slots,
                                    int* n_inputs_used);

/* Launch geometry of the fused elementwise kernels for chains that read n_inputs distinct arrays of n elements
 * (cuda_backend::LaunchConfig::elementwise, rust-engine/src/cuda_backend.rs:134-141, for this library: a
 * persistent grid, 256 consumer threads + one producer warp per CTA, a shared-memory ring). Host only. */
int symplex_b200_fused_elementwise_plan(int n_inputs, int64_t n, int element_bytes, int num_sms,
                                        int32_t grid_dims[3], int32_t block_dims[3], int32_t* shared_mem_bytes);

/* ---- planning queries (host only, no GPU needed) ----------------------------------------------- */

/* hardware::HardwareTarget::B200() (include/symplex/hardware/hardware_target.h:303-329) with the figures of the
 * real part: 148 SMs (the reference says 160), 228 KB shared memory and 256 KB tensor memory per SM, the
 * tcgen05.mma atom 128 x 256 x 16 for bf16 (256 rows for a CTA pair; the reference assumes the 16 x 8 x 32
 * warp-level mma), measured HBM copy bandwidth and bf16 throughput next to the nominal ones. num_sms is read
 * from the current device when one is present (from_device = 1). */
typedef struct symplex_b200_target {
  int32_t num_sms, warp_size, max_warps_per_sm, max_threads_per_sm;
  int32_t shared_mem_bytes_per_sm, max_shared_mem_per_block, register_file_bytes_per_sm, tensor_memory_bytes_per_sm;
  int32_t max_registers_per_thread, num_fp32_lanes_per_sm;
  int32_t mma_m, mma_n, mma_k, mma_pair_m;
  char mma_dtype[8];
  double global_bw_gbps, global_bw_nominal_gbps;
  double bf16_dense_tflops, bf16_dense_tflops_sustained, bf16_dense_tflops_nominal;
  double global_capacity_gb;
  int32_t l2_cache_kb;
  double nvlink_gbps_per_direction;
  int32_t has_tma, has_async_copy, has_tensor_memory, pipeline_stages, from_device;
} symplex_b200_target;
int symplex_b200_hardware_target(symplex_b200_target* out);

/* poly_get_micro_kernel_config (rust-engine/src/ffi.rs:695-717; table in rust-engine/src/polyhedral.rs:4375-4422).
 * target 0 ServerX86, 1 EdgeDevice, 2 TensorAccelerator answer exactly as the reference does; target 3 = B200
 * answers with what this library's kernels use: the tcgen05.mma atom (128 x 256 x 16 for 2-byte elements,
 * 128 x 128 x 8 for tf32), the accumulator size in tensor-memory columns, and the pipeline depth - 1 as the
 * prefetch distance. Null output pointers are skipped. */
void symplex_b200_micro_kernel_config(uint8_t target, size_t element_bytes, size_t* out_tile_m, size_t* out_tile_n,
                                      size_t* out_tile_k, size_t* out_acc_regs, size_t* out_prefetch_dist);

/* training::CompilerPipeline::compile_matmul -> PipelineResult (include/symplex/training/compiler_pipeline.h:18-33,70)
 * and cuda_backend::LaunchConfig::matmul (rust-engine/src/cuda_backend.rs:144-154) for this library: which
 * precompiled kernel a descriptor dispatches to, its tile, launch geometry, shared / tensor memory, scratch need,
 * and a latency estimate from the measured roofline. There is no ptx_source: nothing is generated at run time.
 * The decision is made by the same function the launch path uses. num_sms <= 0 means 148. */
typedef struct symplex_gemm_plan {
  char kernel_name[64];
  int32_t tile_m, tile_n, tile_k;      /* output tile per CTA (per CTA pair if cluster_size == 2), K per stage */
  int32_t mma_m, mma_n, mma_k;         /* one tcgen05.mma */
  int32_t cluster_size, stages;
  int32_t grid_dims[3], block_dims[3]; /* persistent grid: min(tiles, SMs) CTAs */
  int32_t shared_mem_bytes, tmem_columns;
  int32_t prepass_launches;            /* operand preparation kernels launched before the GEMM */
  int32_t bound;                       /* 0 tensor, 1 HBM */
  int64_t tiles;
  size_t workspace_bytes;
  double flops, bytes;                 /* 2MNK x batch; operands read once + output written once */
  double estimated_latency_ns, estimated_tflops, speedup_vs_naive;
  int32_t valid;
  char error[128];
} symplex_gemm_plan;
int symplex_b200_gemm_plan(const symplex_gemm_desc* desc, int num_sms, symplex_gemm_plan* out);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* SYMPLEX_B200_H */
