/*
 * symplex_b200 — C ABI of the B200 (sm_100a) dense-matmul kernel library.
 *
 * Everything SympleX's host code (Rust `extern "C"`, pyo3, ctypes, C++) needs in order to run its
 * tiled dense matmul and the elementwise epilogues fused into it on a B200. Plain pointers and sizes
 * only. Unless a function says otherwise it returns 0 on success or one of the negative
 * SYMPLEX_ERR_* codes; nothing throws across this boundary and there is no CPU fallback: without a
 * usable GPU every compute entry point fails with SYMPLEX_ERR_DRIVER. The void entry points, which
 * have no return value, fill C with NaN when they fail for any reason (no device, out of memory, a
 * device-side timeout) and record why: symplex_b200_last_error() reads "no error" after a void entry
 * point that succeeded.
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
#define SYMPLEX_DT_F64 10 /* TensorMatMul records and the f64 thin ABI only; not an in_dtype of symplex_gemm_desc */
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

/* ---- row-sharded GEMM across the GPUs of one box --------------------------------------------- */

/* What one rank knows about the group. The reference only plans this computation
 * (ShardingAnalyzer::analyze_matmul, include/symplex/distributed/sharding.h:107-112; CollectiveOp::ALL_GATHER and
 * NCCLBridge::emit_nccl_ops, include/symplex/distributed/nccl_bridge.h:19-26,91-98, emit the collective as text);
 * this is the handle of the executed counterpart. The host creates, once, on every rank: a full [M, N] C buffer and
 * a flag block of SYMPLEX_B200_COMM_FLAG_WORDS zeroed int32, both in memory that the other ranks can map (CUDA IPC,
 * cuMemExportToShareableHandle, or torch symmetric memory), and fills in the addresses at which THIS process sees
 * every rank's buffers (index = rank; its own entry is its local memory). c_multicast is the address of a multicast
 * mapping of the C buffers (cuMulticastCreate / cuMulticastBindMem), or NULL. Zero the flags and epoch before the
 * first call and let every rank finish that (a host barrier) before any rank calls symplex_b200_sharded_gemm. */
#define SYMPLEX_B200_MAX_RANKS 8
#define SYMPLEX_B200_COMM_FLAG_WORDS 16
typedef struct symplex_b200_comm {
  int32_t rank, world;
  void* c_base[SYMPLEX_B200_MAX_RANKS];
  void* c_multicast;
  int32_t* flags[SYMPLEX_B200_MAX_RANKS];
  int64_t epoch;         /* collective calls made so far; maintained by the library */
  int32_t wait_limit_ms; /* bound of every device-side wait for a peer; 0 = 2000 */
  int32_t reserved;
} symplex_b200_comm;

/* How C travels. UNICAST: forwarder warps of the GEMM kernel copy each finished tile from the local C to every
 * peer's C with 16-byte stores over NVLink. MULTICAST: the same warps store each tile once to c_multicast and the
 * NVSwitch delivers it to every GPU (multimem.st). EPILOGUE_TMA: the epilogue warps forward their own blocks by TMA
 * (the first design; kept for comparison) - this mode does NOT order the ranks, the caller must (all ranks idle
 * before the call, all ranks done before C is read). AUTO picks UNICAST. */
#define SYMPLEX_XCHG_AUTO 0
#define SYMPLEX_XCHG_UNICAST 1
#define SYMPLEX_XCHG_MULTICAST 2
#define SYMPLEX_XCHG_EPILOGUE_TMA 3

/* C = act(alpha * A.B + bias) with the rows of A and C split evenly over comm->world ranks (rank r owns rows
 * [r * M / world, (r + 1) * M / world)), B replicated, and C all-gathered: when the kernel this call enqueues on
 * `stream` has finished, comm->c_base[rank] holds the whole [M, N] product. One kernel per rank does the GEMM and
 * the exchange; the ranks order themselves with flags in each other's memory (UNICAST / MULTICAST): a rank's C is
 * not overwritten before it has entered the call, and the kernel does not end before every peer's tiles have
 * landed. d describes the GLOBAL problem (d->M = all rows; bf16 inputs for world > 1; batch 1; dense C). Collective:
 * every rank calls it, the same number of times, in the same order. A peer that does not show up within the wait
 * limit makes the kernel give up: symplex_b200_sync_status then returns SYMPLEX_ERR_TIMEOUT on the ranks that
 * waited, and C is not valid. */
int symplex_b200_sharded_gemm(const symplex_gemm_desc* d, const void* A_local, const void* B, const float* bias,
                              symplex_b200_comm* comm, int32_t exchange, void* stream);

/* ShardingAnalyzer::analyze_matmul -> ShardPlan (include/symplex/distributed/sharding.h:65-112) as plain data, for
 * the row split this library executes: A SHARD_DIM_0, B REPLICATE, C SHARD_DIM_0 followed by an all-gather.
 * Strategy codes are the reference's ShardingStrategy values (sharding.h:18-24). Returns SYMPLEX_ERR_INVALID if M
 * does not split evenly. Host only. */
typedef struct symplex_shard_spec {
  int32_t strategy;         /* 0 REPLICATE, 1 SHARD_DIM_0, ... */
  int32_t shard_dim;        /* -1 if replicated */
  int64_t original_shape[2], local_shape[2];
} symplex_shard_spec;
typedef struct symplex_shard_plan {
  symplex_shard_spec a, b, c;
  int32_t n_all_gather_ops; /* 1 if world > 1: all_gather(C, dim 0) */
  int32_t n_all_reduce_ops, n_all_to_all_ops; /* 0 */
  int32_t world;
  int64_t total_communication_bytes; /* received by all devices together: world * (world - 1) * M/world * N * bytes */
  int64_t peak_memory_per_device;    /* local A + B + full C */
} symplex_shard_plan;
int symplex_b200_analyze_matmul(int64_t M, int64_t N, int64_t K, int32_t world, int32_t bytes_per_element,
                                symplex_shard_plan* out);

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
 * on it and must be serialised by the caller. Nothing needs clearing between calls. "No allocating routine" is
 * about this library's code: the first CUDA call of a process on a device creates its context and loads the
 * library's kernels, and that is also when the array becomes resident. A device-side failure (a bounded wait
 * that ran out) is reported by symplex_b200_noalloc_status, below - not by symplex_b200_sync_status. */
#define SYMPLEX_B200_NOALLOC_SCRATCH_BYTES (16 * 1024 * 1024)
int symplex_b200_sgemm_noalloc(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                               void* stream);

/* Status of the symplex_b200_sgemm_noalloc calls since the last call of this function on the current device:
 * synchronises `stream`, returns 0 or SYMPLEX_ERR_TIMEOUT (a bounded device-side wait ran out; C of those calls
 * is not valid) and clears the word. No counterpart in the reference. Like the entry point it serves, it calls no
 * allocating routine: the status word is a second small variable inside the library image, read with a plain
 * device-to-host copy into a stack variable. (symplex_b200_sync_status reports the other entry points' status word
 * and may allocate on its first call; it does not see a no-alloc failure.) */
int symplex_b200_noalloc_status(void* stream);

/* Synchronise `stream` and return the device-side status of the launches since the last call:
 * 0, SYMPLEX_ERR_TIMEOUT or SYMPLEX_ERR_EXEC. */
int symplex_b200_sync_status(void* stream);

/* Self-test of the kernels' unwinding: runs one 128 x 64 x 128 bf16 product (A [128,128], B [128,64] row-major,
 * C [128,64] bf16, device pointers) in which the TMA producer deliberately leaves out the last k-block and every
 * wait is bounded by limit_ms (1..1000). The MMA thread's wait for that block runs out, every role of the CTA
 * unwinds (copies drained, tensor memory freed) and the kernel returns normally with its status word set.
 * Synchronises, clears the status word and returns what it found: SYMPLEX_ERR_TIMEOUT is the expected result,
 * 0 means the wait did not run out. Nothing traps and nothing spins without a bound; the next call on the device
 * works as usual. No counterpart in the reference. */
int symplex_b200_selftest_wait_timeout(const void* A, const void* B, void* C, int32_t limit_ms, void* stream);

/* Process-wide tuning overrides, for tests and experiments: "tile_n" (0 auto, 64/128/256), "pair_mode" (-1 auto,
 * 0 single-CTA tiles, 1 256x256 CTA pairs, 2 512x256 CTA pairs), "stream_k" (0; 1: bf16 problems take the 512x256 pairs with
 * the k-blocks of all tiles shared evenly among them instead of whole tiles, wherever the library's own scratch pool
 * serves the call - measured no faster than whole tiles on B200, hence off; "stream_k_launches" counts such launches), "f32_fused" (-1 auto, 0, 1), "f32_split_k" (0 auto,
 * 1, 2, 4), "f32_tile_rows" (0 auto, 128), "group_m" (0 auto), "tma_store" (1, 0), "pipeline_mb" (96),
 * "pipeline" (1, 0), "wait_limit_ms" (2000), "pdl" (1, 0: the GEMM kernels start their set-up while the kernel before
 * them in the stream drains, and wait for it before touching memory), "trace" (0, 1: one line per GEMM dispatch on stderr). Only "tile_n"
 * and "trace" can also be preset from the environment (SYMPLEX_B200_TILE, SYMPLEX_B200_TRACE, read once at load);
 * the pipeline depth is a compile-time constant of each kernel. set returns SYMPLEX_ERR_INVALID for an unknown
 * name; get returns INT64_MIN for one. */
int symplex_b200_set_option(const char* name, int64_t value);
int64_t symplex_b200_get_option(const char* name);

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
/* Their f64 twins (rust-engine/src/phase3_jit.rs:449-461,676-685), which TensorMatMul traces with element type F64
 * call (:13024-13118): C = A.B in double precision, host pointers, row-major. Computed by a CUDA-core kernel in
 * the summation order of the reference's cache_tiled_dgemm (:578-650: per block of 128 consecutive k a chain of
 * separately rounded multiply and add from 0, blocks added to C in increasing k), so the results are bit-identical
 * to that function's (a CBLAS build of the reference, which rounds differently, agrees to ~1e-15). */
void blas_dgemm(const double* a, const double* b, double* c, size_t m, size_t n, size_t k);
void cache_tiled_dgemm_thin(const double* a, const double* b, double* c, size_t m, size_t n, size_t k);
/* The same product on device pointers, asynchronous on `stream`; lda / ldb / ldc in elements (0 = packed). */
int symplex_b200_dgemm(const double* A, const double* B, double* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                       int64_t ldb, int64_t ldc, void* stream);

/* Execute one serialized Instr::TensorMatMul record (rust-engine/src/types.rs:407-417,646-657,884-904: opcode
 * 0xA2, dst/lhs/rhs slot u16, m/n/k u64, element_ty, lhs_layout, rhs_layout; 34 bytes little endian) against an
 * array of host pointers indexed by slot - what the reference's JIT lowers to a blas_sgemm call
 * (rust-engine/src/phase3_jit.rs:13024-13118). Unlike the reference, which parses the layout bytes and then
 * ignores them, rhs_layout is honoured (RowMajor: [K,N]; ColMajor: stored [N,K]); F32 and BF16 element types, and
 * F64 (row-major rhs only; the product blas_dgemm computes); lhs must be RowMajor. Returns 0 or a negative
 * SYMPLEX_ERR_* code. */
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
/* The same list continued: ..., symplex_b200_comm, symplex_shard_plan, symplex_generated_kernel, symplex_fusion_op,
 * symplex_kernel_args. Writes the first n entries to out (may be NULL) and returns how many there are. */
int32_t symplex_b200_abi_sizes_ext(int32_t* out, int32_t n);

/* Stream-K work list of CTA pair `pair` of `pairs` for `tiles` output tiles of `k_blocks` k-blocks each, computed on the
 * host by the iterator the kernel runs (no GPU needed; for tests and tools). items receives up to cap entries of
 * {tile, first k-block, end k-block, kind} with kind 0 = whole tile, 1 = partial sums left for the tile's owner,
 * 2 = owner (holds the tile's last k-block, adds the partial sums of contributors[i] lower-numbered pairs). Returns the
 * number of items the pair has, or -1 for invalid arguments. */
int32_t symplex_b200_stream_k_items(int32_t pair, int32_t pairs, int32_t tiles, int32_t k_blocks, int32_t* items,
                                    int32_t cap, int32_t* contributors);

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
/* The same function under the reference's own symbol name and argument list
 * (include/symplex/polyhedral/rust_bridge.h:221-229, rust-engine/src/ffi.rs:695-717), so C++ code that declares
 * it extern "C" links against this library unchanged. */
void poly_get_micro_kernel_config(uint8_t target, size_t element_bytes, size_t* out_tile_m, size_t* out_tile_n,
                                  size_t* out_tile_k, size_t* out_acc_regs, size_t* out_prefetch_dist);

/* codegen::CodeGenerator::generate_matmul(M, N, K, TileConfig, depth) -> GeneratedKernel
 * (include/symplex/codegen/code_generator.h:19-45) for a library of precompiled kernels: the kernel a bf16 (element
 * bytes 2) or fp32 (4) product of that shape dispatches to, its launch geometry and resource use. The TileConfig's
 * tile_n is taken as the advisory hint of symplex_gemm_desc (0 / 64 / 128 / 256; other values are ignored, as the
 * reference's generator repairs infeasible tiles). There is no ptx_source. register_count is the per-thread
 * register budget the kernel is compiled for (64K registers / threads per CTA). valid = 0 and error_message set for
 * an empty problem. Host only. */
typedef struct symplex_generated_kernel {
  char kernel_name[64];
  int64_t shared_mem_bytes, register_count;
  int64_t grid_dims[3], block_dims[3];
  int32_t valid;
  char error_message[128];
} symplex_generated_kernel;
int symplex_b200_generate_matmul(int64_t M, int64_t N, int64_t K, int32_t element_bytes, int64_t tile_m, int64_t tile_n,
                                 int64_t tile_k, symplex_generated_kernel* out);

/* ---- fusion discovery for the matmul path (host only) -------------------------------------------- */

/* One op as the reference's discover_fusions takes it (rust-engine/src/lib.rs:344-348): name ("matmul",
 * "batch_matmul", "add", "mul", "relu", "gelu", "sigmoid", "tanh", "silu", ...; others never fuse into a matmul),
 * output shape, dtype name ("fp32", "fp16", "bf16", "fp8", "int8", "int4"; unknown = fp32). */
typedef struct symplex_fusion_op {
  const char* op;
  const int64_t* shape;
  int32_t rank;
  const char* dtype;
} symplex_fusion_op;

/* symplex_engine.discover_fusions (rust-engine/src/lib.rs:344-413) restricted to the one pattern of this path:
 * every maximal chain [matmul, (mul,) (add,) (activation)] of at least two ops that
 * matches_matmul_bias_activation accepts (rust-engine/src/fusion_engine.rs:1587-1623) becomes one
 * "MatMulBiasReLU" boundary with estimate_memory_savings' traffic figure (:1209-1225: 2 x bytes(op 0) +
 * 2 x bytes(op 1)), compute_savings_factor 1.1 and the pattern's base confidence 0.9. Writes the JSON document of
 * the reference's schema into json_out (NUL terminated) and returns its length, or the negated length needed if
 * cap is too small (nothing is written then), or SYMPLEX_ERR_INVALID for null arguments. */
int64_t symplex_b200_discover_fusions(const symplex_fusion_op* ops, size_t n_ops, char* json_out, size_t cap);

/* The longest prefix of ops[first..] that one GEMM launch executes, written into the epilogue fields of *d:
 * [matmul, (mul,) (add,) (activation)] -> act(alpha * A.B + bias). Sets d->activation; *consumed = ops used
 * (1 = a bare matmul), *has_bias / *has_scale say whether the caller must pass a bias vector / set d->alpha to the
 * multiplier. Returns SYMPLEX_ERR_INVALID if ops[first] is not a matmul. */
int symplex_b200_compile_epilogue(const symplex_fusion_op* ops, size_t n_ops, size_t first, symplex_gemm_desc* d,
                                  int32_t* consumed, int32_t* has_bias, int32_t* has_scale);

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
