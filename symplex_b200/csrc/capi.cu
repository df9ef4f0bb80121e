// C-ABI layer of libsymplex_b200.so: descriptor validation, scratch planning, operand preparation,
// kernel dispatch, and the host-pointer drop-ins for the reference's matmul entry points.
// Declarations and the reference interfaces they replace: include/symplex_b200.h.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <memory>
#include <mutex>

#include "../../include/symplex_b200.h"
#include "gemm_params.h"
#include "host_api.h"
#include "options.h"

namespace sx {

// ------------------------------------------------------------------ options
Options& options() {
  static Options o;
  static const bool init = [] {
    if (const char* e = getenv("SYMPLEX_B200_TILE")) o.tile_n = atoi(e);
    if (const char* e = getenv("SYMPLEX_B200_TRACE")) o.trace = atoi(e);
    return true;
  }();
  (void)init;
  return o;
}

bool pdl_enabled() { return options().pdl.load(std::memory_order_relaxed) != 0; }

static std::atomic<int64_t>* option_by_name(const char* name) {
  if (name == nullptr) return nullptr;
  Options& o = options();
  struct Entry { const char* name; std::atomic<int64_t>* v; };
  const Entry table[] = {
      {"tile_n", &o.tile_n}, {"pair_mode", &o.pair_mode}, {"stream_k", &o.stream_k}, {"f32_fused", &o.f32_fused},
      {"f32_split_k", &o.f32_split_k}, {"f32_tile_rows", &o.f32_tile_rows}, {"group_m", &o.group_m},
      {"tma_store", &o.tma_store}, {"pipeline_mb", &o.pipeline_mb}, {"pipeline", &o.pipeline},
      {"wait_limit_ms", &o.wait_limit_ms}, {"pdl", &o.pdl}, {"trace", &o.trace}, {"stream_k_launches", &o.stream_k_launches},
  };
  for (const Entry& e : table)
    if (strcmp(e.name, name) == 0) return e.v;
  return nullptr;
}

// ------------------------------------------------------------------ errors / counters
static thread_local char g_err[512] = "no error";
static std::atomic<uint64_t> g_launches{0};

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// For the other translation units of the library: record a message for symplex_b200_last_error().
int set_last_error(int code, const char* msg) { return fail(code, "%s", msg); }

static int cuda_fail(cudaError_t e, const char* what) {
  const int code = (e == cudaErrorMemoryAllocation) ? SX_ERR_OOM
                   : (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver || e == cudaErrorInitializationError)
                       ? SX_ERR_DRIVER
                       : SX_ERR_EXEC;
  return fail(code, "%s: %s", what, cudaGetErrorString(e));
}

#define SX_CUDA(call)                                   \
  do {                                                  \
    cudaError_t e__ = (call);                           \
    if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
  } while (0)

// ------------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess ||
        qr != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int encode_tensor_map_3d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, const uint64_t dims[3],
                         const uint64_t strides_bytes[2], const uint32_t box[3], bool swizzle128) {
  // A tensor map is a pure function of the address and geometry it is encoded from, and callers in a loop pass
  // the same few operands again and again, so the last encodes of this thread are kept (direct-mapped, no lock).
  struct Cached {
    uint64_t key[9];
    CUtensorMap map;
    bool valid;
  };
  constexpr int CACHE_SLOTS = 32;
  static thread_local Cached cache[CACHE_SLOTS] = {};
  const uint64_t key[9] = {reinterpret_cast<uint64_t>(base), dims[0], dims[1], dims[2], strides_bytes[0],
                           strides_bytes[1], (uint64_t(box[0]) << 32) | box[1],
                           (uint64_t(box[2]) << 32) | (uint64_t(dt) << 1) | (swizzle128 ? 1u : 0u), 0};
  uint64_t h = 0x9e3779b97f4a7c15ull;
  for (int i = 0; i < 8; ++i) h = (h ^ key[i]) * 0xff51afd7ed558ccdull;
  Cached& slot = cache[(h >> 40) % CACHE_SLOTS];
  if (slot.valid && memcmp(slot.key, key, sizeof(key)) == 0) {
    *out = slot.map;
    return SX_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(SX_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t d[3] = {dims[0], dims[1], dims[2]};
  cuuint64_t s[2] = {strides_bytes[0], strides_bytes[1]};
  cuuint32_t b[3] = {box[0], box[1], box[2]};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(SX_ERR_INVALID, "cuTensorMapEncodeTiled failed (%d): dims %llu,%llu,%llu strides %llu,%llu box %u,%u,%u",
                (int)r, (unsigned long long)d[0], (unsigned long long)d[1], (unsigned long long)d[2],
                (unsigned long long)s[0], (unsigned long long)s[1], b[0], b[1], b[2]);
  memcpy(slot.key, key, sizeof(key));
  slot.map = *out;
  slot.valid = true;
  return SX_OK;
}

// ------------------------------------------------------------------ per-device state
struct DeviceState {
  std::mutex mu;
  bool ready = false;
  int num_sms = 0;
  int* status = nullptr;  // device word written by kernels that unwind
  unsigned* xchg_counter = nullptr;  // device word of the sharded GEMM's forwarder warps (zero between launches)
  int* sk_flags = nullptr;           // stream-K flag words of the pair kernel (zeroed once, then compared with sk_epoch)
  int sk_epoch = 0;                  // stream-K launches so far on this device; advanced under `mu`
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  cudaEvent_t scratch_free = nullptr;  // recorded after the last launch that reads the pooled scratch
  cudaStream_t scratch_stream = nullptr;  // the stream that launch went to
  bool scratch_used = false;
  char* fe_scratch = nullptr;  // FE_SCRATCH_SETS reduction scratch areas of the fused elementwise kernels
  std::atomic<unsigned> fe_next{0};
};
static DeviceState g_dev[16];
constexpr int FE_SCRATCH_SETS = 8;

static int device_state(DeviceState** out) {
  int dev = 0;
  SX_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 16) return fail(SX_ERR_INVALID, "device ordinal %d out of range", dev);
  DeviceState& st = g_dev[dev];
  std::lock_guard<std::mutex> lk(st.mu);
  if (!st.ready) {
    int major = 0;
    SX_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return fail(SX_ERR_DRIVER, "device %d is sm_%d0, this library needs sm_100", dev, major);
    SX_CUDA(cudaDeviceGetAttribute(&st.num_sms, cudaDevAttrMultiProcessorCount, dev));
    SX_CUDA(cudaMalloc(&st.status, 64));
    SX_CUDA(cudaMemset(st.status, 0, 64));
    st.xchg_counter = reinterpret_cast<unsigned*>(st.status) + 8;
    SX_CUDA(cudaMalloc(&st.sk_flags, stream_k_flag_words(st.num_sms) * sizeof(int)));
    SX_CUDA(cudaMemset(st.sk_flags, 0, stream_k_flag_words(st.num_sms) * sizeof(int)));
    SX_CUDA(cudaEventCreateWithFlags(&st.scratch_free, cudaEventDisableTiming));
    SX_CUDA(cudaMalloc(&st.fe_scratch, FE_SCRATCH_SETS * FE_REDUCE_SCRATCH_BYTES));
    SX_CUDA(cudaMemset(st.fe_scratch, 0, FE_SCRATCH_SETS * FE_REDUCE_SCRATCH_BYTES));
    st.ready = true;
  }
  *out = &st;
  return SX_OK;
}

// Where a launch gets its scratch from. Three sources: a pointer the caller owns (symplex_b200_gemm_ws, the
// host-pointer paths' per-thread buffer), nothing, or the grow-only pool of the device. The pool is one block
// shared by every caller of symplex_b200_gemm on that device, so its users are serialised: the pool's mutex is
// held from the moment the pointer is handed out until the launches that use it have been enqueued (no other
// thread can grow - and free - the block in between), and an event recorded after those launches makes a later
// user on ANOTHER stream wait for them on the GPU. Growing synchronises the device before it frees the old
// block. While `stream` is being captured into a CUDA graph no event is recorded or awaited (the capture's own
// dependencies order the nodes; a graph that is replayed next to other pooled-scratch users is the caller's to
// order).
static int host_buf(int i, size_t bytes, void** out);

struct Scratch {
  void* fixed = nullptr;
  DeviceState* pool = nullptr;
  cudaStream_t stream = nullptr;
  bool locked = false, capturing = false, host_thread = false;

  static Scratch from_pointer(void* p) {
    Scratch s;
    s.fixed = p;
    return s;
  }
  // the calling thread's own grow-only buffer (host-pointer paths), allocated when a kernel first needs it
  static Scratch from_host_thread() {
    Scratch s;
    s.host_thread = true;
    return s;
  }
  static Scratch from_pool(DeviceState* st, cudaStream_t stream) {
    Scratch s;
    s.pool = st;
    s.stream = stream;
    return s;
  }
  Scratch() = default;
  Scratch(const Scratch&) = delete;
  Scratch& operator=(const Scratch&) = delete;
  Scratch(Scratch&& o) noexcept
      : fixed(o.fixed), pool(o.pool), stream(o.stream), locked(o.locked), capturing(o.capturing), host_thread(o.host_thread) {
    o.locked = false;
  }

  int get(size_t bytes, void** out) {
    if (host_thread) return host_buf(6, bytes, out);
    if (pool == nullptr) {
      *out = fixed;
      return SX_OK;
    }
    DeviceState* st = pool;
    if (!locked) {
      st->mu.lock();
      locked = true;
      cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
      if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) cudaGetLastError();
      capturing = cs != cudaStreamCaptureStatusNone;
    }
    if (bytes > st->scratch_bytes) {
      if (st->scratch) {
        SX_CUDA(cudaDeviceSynchronize());
        SX_CUDA(cudaFree(st->scratch));
        st->scratch = nullptr;
        st->scratch_bytes = 0;
        st->scratch_used = false;
      }
      const size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
      SX_CUDA(cudaMalloc(&st->scratch, want));
      st->scratch_bytes = want;
    }
    if (!capturing && st->scratch_used && st->scratch_stream != stream)
      SX_CUDA(cudaStreamWaitEvent(stream, st->scratch_free, 0));
    *out = st->scratch;
    return SX_OK;
  }

  ~Scratch() {
    if (!locked) return;
    if (!capturing) {
      if (cudaEventRecord(pool->scratch_free, stream) == cudaSuccess) {
        pool->scratch_used = true;
        pool->scratch_stream = stream;
      } else {
        cudaGetLastError();
      }
    }
    pool->mu.unlock();
  }
};

// ------------------------------------------------------------------ planning
static inline long long round_up(long long x, long long m) { return (x + m - 1) / m * m; }
static inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

struct Plan {
  long long M, N, K;
  int batch;
  bool f32_in, bf16_out, b_col;
  long long lda, ldb, ldc, a_bs, b_bs, c_bs;
  long long b_rows, b_cols;  // B as stored: [b_rows, b_cols]
  // scratch
  bool a_prep, b_prep;
  long long a_ldp, b_ldp;  // leading dimension of the prepared copies
  size_t a_off, b_off, total;
  bool b_ready = false;  // the prepared copy of B is already in the scratch (row-chunked host path)
};

static int make_plan(const symplex_gemm_desc* d, const void* A, const void* B, Plan* p) {
  if (d == nullptr) return fail(SX_ERR_INVALID, "null descriptor");
  if (d->M < 0 || d->N < 0 || d->K < 0 || d->batch < 0) return fail(SX_ERR_INVALID, "negative dimension");
  if (d->M > 0x7fffffffLL || d->N > 0x7fffffffLL || d->K > 0x7fffffffLL)
    return fail(SX_ERR_INVALID, "dimension exceeds 2^31-1");
  if (d->in_dtype != SYMPLEX_DT_F32 && d->in_dtype != SYMPLEX_DT_BF16)
    return fail(SX_ERR_INVALID, "in_dtype %d not supported (F32=9, BF16=11)", d->in_dtype);
  if (d->out_dtype != SYMPLEX_DT_F32 && d->out_dtype != SYMPLEX_DT_BF16)
    return fail(SX_ERR_INVALID, "out_dtype %d not supported (F32=9, BF16=11)", d->out_dtype);
  if (d->b_layout != SYMPLEX_ROW_MAJOR && d->b_layout != SYMPLEX_COL_MAJOR)
    return fail(SX_ERR_INVALID, "b_layout %d not supported", d->b_layout);
  if (d->activation < SYMPLEX_ACT_NONE || d->activation > SYMPLEX_ACT_SILU)
    return fail(SX_ERR_INVALID, "activation %d not supported", d->activation);
  if (d->tile_n != 0 && d->tile_n != 64 && d->tile_n != 128 && d->tile_n != 256)
    return fail(SX_ERR_INVALID, "tile_n must be 0, 64, 128 or 256");
  p->M = d->M; p->N = d->N; p->K = d->K;
  p->batch = d->batch;
  p->f32_in = d->in_dtype == SYMPLEX_DT_F32;
  p->bf16_out = d->out_dtype == SYMPLEX_DT_BF16;
  p->b_col = d->b_layout == SYMPLEX_COL_MAJOR;
  p->b_rows = p->b_col ? d->N : d->K;
  p->b_cols = p->b_col ? d->K : d->N;
  p->lda = d->lda ? d->lda : d->K;
  p->ldb = d->ldb ? d->ldb : p->b_cols;
  p->ldc = d->ldc ? d->ldc : d->N;
  if (p->lda < d->K || p->ldb < p->b_cols || p->ldc < d->N) return fail(SX_ERR_INVALID, "leading dimension too small");
  p->a_bs = d->a_batch_stride ? d->a_batch_stride : d->M * p->lda;
  p->b_bs = d->b_batch_stride ? d->b_batch_stride : p->b_rows * p->ldb;
  p->c_bs = d->c_batch_stride ? d->c_batch_stride : d->M * p->ldc;
  size_t off = 0;
  if (p->f32_in) {
    p->a_prep = p->b_prep = true;
    p->a_ldp = round_up(d->K, 4);
    p->b_ldp = round_up(d->K, 4);  // B planes are always written as [N][K]
    p->a_off = off;
    off = align256(off + (size_t)p->batch * 2 * d->M * p->a_ldp * 4);
    p->b_off = off;
    off = align256(off + (size_t)p->batch * 2 * d->N * p->b_ldp * 4);
  } else {
    auto misaligned = [](const void* ptr, long long ld, long long bs) {
      return (ld % 8) != 0 || (bs % 8) != 0 || (reinterpret_cast<uintptr_t>(ptr) % 16) != 0;
    };
    p->a_prep = misaligned(A, p->lda, p->a_bs);
    p->b_prep = misaligned(B, p->ldb, p->b_bs);
    p->a_ldp = round_up(d->K, 8);
    p->b_ldp = round_up(p->b_cols, 8);
    p->a_off = off;
    if (p->a_prep) off = align256(off + (size_t)p->batch * d->M * p->a_ldp * 2);
    p->b_off = off;
    if (p->b_prep) off = align256(off + (size_t)p->batch * p->b_rows * p->b_ldp * 2);
  }
  p->total = off;
  return SX_OK;
}

// Which kernel serves a problem. One place decides, for the launch path and for the planning query alike.
enum KernelKind { KK_F32_FUSED, KK_F32_SPLIT, KK_BF16_TC, KK_BF16_PAIR256, KK_BF16_PAIR512 };
struct KernelChoice {
  KernelKind kind;
  int bn;  // tile width of the single-CTA kernels
  bool stream_k = false;  // KK_BF16_PAIR512 only
};

// sk_ok: the caller can give the 512 x 256 pair kernel its stream-K workspace (pooled scratch, no peers).
static KernelChoice choose_kernel(const Plan& p, int tile_n, int num_sms, int n_peers, bool f32_fused_ok,
                                  bool sk_ok = false) {
  const Options& opt = options();
  int forced = tile_n;
  if (opt.tile_n.load(std::memory_order_relaxed) != 0) forced = (int)opt.tile_n.load(std::memory_order_relaxed);
  if (p.f32_in) {
    // Small and batched problems (each operand element feeds only a few tiles): split inside the GEMM kernel.
    // With at most 64 rows there is a single row of tiles: no B element is converted twice, whatever N is.
    bool fused = (p.M <= 64 || ((p.M + 127) / 128 <= 8 && (p.N + 63) / 64 <= 16)) && f32_fused_ok;
    if (opt.f32_fused.load(std::memory_order_relaxed) >= 0) fused = opt.f32_fused.load(std::memory_order_relaxed) != 0 && f32_fused_ok;
    if (fused) return {KK_F32_FUSED, 64};
    if (forced == 64 || forced == 128) return {KK_F32_SPLIT, forced};
    const bool wide = p.N > 64 && ((p.M + 127) / 128) * ((p.N + 127) / 128) * p.batch >= num_sms;
    return {KK_F32_SPLIT, wide ? 128 : 64};
  }
  const int bn = pick_bn(p.M, p.N, p.batch, num_sms, forced);
  // Tile shape by estimated cost = waves x (output area one SM computes per tile) / tensor-pipe utilisation of the
  // shape, measured on large problems: single-CTA tiles 128 x 256 / 128 / 64 reach 0.70 / 0.56 / 0.40, 256x256 pair
  // tiles 0.80, 512x256 pair tiles 0.875 (least L2 -> SM traffic per flop). Examples (measured): 4096^3 runs 2 waves
  // of 512x256 (108 us) rather than 4 of 256x256 (116 us); 2048^3 one wave of 256x256 pairs (19.6 us) rather than
  // two of 128x128 (28.4 us).
  int mode = 0;  // 0 single CTA, 1 pair 256x256, 2 pair 512x256
  bool stream_k = false;
  if (forced == 0 && p.M > 128 && p.N >= 256) {
    const long long pairs = num_sms / 2;
    const long long nt = (p.N + 255) / 256;
    const long long t0 = ((p.M + 127) / 128) * ((p.N + bn - 1) / bn) * p.batch;
    const long long t256 = ((p.M + 255) / 256) * nt * p.batch, t512 = ((p.M + 511) / 512) * nt * p.batch;
    const double eff0 = bn == 256 ? 0.70 : bn == 128 ? 0.56 : 0.40;
    const double cost0 = (double)((t0 + num_sms - 1) / num_sms) * (128.0 * bn) / eff0;
    const double cost256 = (double)((t256 + pairs - 1) / pairs) * (128.0 * 256.0) / 0.80;
    double cost512 = p.M > 256 ? (double)((t512 + pairs - 1) / pairs) * (256.0 * 256.0) / 0.875 : 1e300;
    // Stream-K (the pairs share the k-blocks of all tiles evenly) is built and tested but never chosen by itself:
    // measured process by process on shapes whose last wave is mostly idle, it is within +-4 % of the better of the
    // two whole-tile shapes (4608 x 4608 x 4096, 2.19 waves: 0.134 ms against 0.138 on whole 512 x 256 tiles and 0.134
    // on 256 x 256 tiles; 8192 x 4864 x 8192, 4.11 waves: 0.481 against 0.476; sustained runs under the power cap:
    // 0.549 against 0.534). These GEMMs are bound by what the whole chip shares - the L2 -> SM path at burst clocks,
    // the power limit in long runs - so pairs that idle in the last wave cost far less than their share, and the
    // extra L2 traffic of stream-K (partial sums, operand requests that no longer coincide) eats the rest.
    // The option stream_k = 1 takes it wherever it can run.
    const long long nkb = (p.K + 63) / 64;
    const long long sk_setting = opt.stream_k.load(std::memory_order_relaxed);
    if (sk_ok && sk_setting > 0 && n_peers == 0 && p.M > 256 && t512 * nkb >= pairs * 16 && t512 * nkb <= 0x7fffffffLL) {
      cost512 = 0.0;
      stream_k = true;
    }
    if (cost512 <= cost256 && cost512 <= cost0) mode = 2;
    else if (cost256 <= cost0) mode = 1;
  }
  // Row-sharded products whose exchange takes longer than their math (inbound bytes at the measured peer-copy
  // rate against the flops at the kernel's sustained rate): the link is the critical path from the first finished
  // tile to the last, so the 256 x 256 tiles, whose first tile is ready in half the time, beat the wider tile's better
  // tensor-pipe utilisation.
  if (n_peers > 0 && mode == 2) {
    const double compute_s = 2.0 * (double)p.M * (double)p.N * (double)p.K / (1663.5e12 * 0.85);
    const double link_s = (double)p.M * (double)p.N * (p.bf16_out ? 2.0 : 4.0) * n_peers / 770e9;
    if (link_s > compute_s) mode = 1;
  }
  if (opt.pair_mode.load(std::memory_order_relaxed) >= 0) mode = (int)opt.pair_mode.load(std::memory_order_relaxed);
  if (n_peers > 0 && mode == 0) mode = 1;  // only the pair kernels carry the peer-store epilogue
  return {mode == 2 ? KK_BF16_PAIR512 : mode == 1 ? KK_BF16_PAIR256 : KK_BF16_TC, bn, stream_k && mode == 2};
}

// Peer destinations of a launch (row-sharded products); see Exchange in gemm_params.h.
struct PeerArgs {
  int n_peers = 0;
  int xchg = 0;  // 0: XCHG_EPILOGUE_TMA when n_peers > 0
  const void* peer_C[7] = {};
  int my_rank = 0, peer_rank[7] = {};
  void* mc_C = nullptr;
  int* flags = nullptr;
  int* peer_flags[7] = {};
  int epoch = 0;
  unsigned long long wait_limit_ns = 0;
};

static int run_gemm(const symplex_gemm_desc* d, const Plan& p, const void* A, const void* B, void* C,
                    const float* bias, const void* residual, Scratch& scratch, DeviceState* st, cudaStream_t stream,
                    const PeerArgs* peers = nullptr) {
  if (p.M == 0 || p.N == 0 || p.batch == 0) return SX_OK;  // nothing to write
  if (p.K == 0) return fail(SX_ERR_INVALID, "K == 0 is not supported by the device entry points");
  const Options& opt = options();
  const int n_peers = peers ? peers->n_peers : 0;
  uint8_t* w = nullptr;
  // The kernel of a bf16 product is chosen before any scratch is taken: stream-K adds its workspace behind the
  // prepared operand copies, and the pooled block must be asked for once, at its full size.
  KernelChoice kc{};
  size_t sk_bytes = 0;
  if (!p.f32_in) {
    kc = choose_kernel(p, d->tile_n, st->num_sms, n_peers, false, scratch.pool != nullptr);
    if (kc.stream_k) sk_bytes = stream_k_workspace_bytes(st->num_sms);
  }
  const size_t sk_off = align256(p.total);
  auto need_scratch = [&]() -> int {
    const size_t want = sk_bytes ? sk_off + sk_bytes : p.total;
    if (w != nullptr || want == 0) return SX_OK;
    void* ws = nullptr;
    int rc = scratch.get(want, &ws);
    if (rc != SX_OK) return rc;
    if (ws == nullptr) return fail(SX_ERR_INVALID, "this problem needs %zu bytes of scratch", want);
    w = static_cast<uint8_t*>(ws);
    return SX_OK;
  };
  TcGemmArgs g{};
  g.M = p.M; g.N = p.N; g.batch = p.batch;
  g.out_bf16 = p.bf16_out;
  g.b_mn = !p.b_col;
  g.C = C; g.ldc = p.ldc; g.c_batch_stride = p.c_bs;
  g.bias = bias; g.residual = residual;
  g.alpha = d->alpha; g.beta = d->beta; g.act = d->activation;
  g.status = st->status;
  g.num_sms = st->num_sms;
  g.K = p.K;
  g.wait_limit_ns = (unsigned long long)opt.wait_limit_ms.load(std::memory_order_relaxed) * 1000000ull;
  if (peers && peers->wait_limit_ns) g.wait_limit_ns = peers->wait_limit_ns;
  g.group_m = (int)opt.group_m.load(std::memory_order_relaxed);
  if (n_peers > 0 && p.f32_in)
    return fail(SX_ERR_INVALID, "peer destinations are supported for bf16 inputs only");
  int rc;
  if (p.f32_in) {
    // Small and batched problems (each operand element feeds only a few tiles): split inside the GEMM kernel.
    {
      TcGemmArgs f = g;
      f.b_mn = !p.b_col;
      f.A = A; f.lda = p.lda; f.a_plane_stride = p.a_bs;
      f.B = B; f.ldb = p.ldb; f.b_plane_stride = p.b_bs;
      if (choose_kernel(p, d->tile_n, st->num_sms, 0, f32_fused_operands_ok(f)).kind == KK_F32_FUSED) {
        if (opt.trace.load(std::memory_order_relaxed))
          fprintf(stderr, "[symplex_b200] gemm %lldx%lldx%lld batch %d f32 -> in-kernel-split kernel\n", p.M, p.N, p.K, p.batch);
        rc = launch_gemm_f32_fused(f, stream);
        if (rc == SX_ERR_EXEC) return fail(rc, "GEMM kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        if (rc != SX_OK) return rc;
        ++g_launches;
        return SX_OK;
      }
    }
    // Otherwise both operands are rewritten as {hi, lo} tf32 planes with K contiguous.
    if ((rc = need_scratch()) != SX_OK) return rc;
    float* Ap = reinterpret_cast<float*>(w + p.a_off);
    float* Bp = reinterpret_cast<float*>(w + p.b_off);
    rc = launch_split_tf32(static_cast<const float*>(A), p.lda, p.a_bs, Ap, (int)p.M, (int)p.K, (int)p.a_ldp,
                           p.batch, stream);
    if (rc != SX_OK) return fail(rc, "split_tf32(A) launch failed");
    ++g_launches;
    if (!p.b_ready) {
      if (p.b_col)
        rc = launch_split_tf32(static_cast<const float*>(B), p.ldb, p.b_bs, Bp, (int)p.N, (int)p.K, (int)p.b_ldp,
                               p.batch, stream);
      else
        rc = launch_split_tf32_transpose(static_cast<const float*>(B), p.ldb, p.b_bs, Bp, (int)p.K, (int)p.N,
                                         (int)p.b_ldp, p.batch, stream);
      if (rc != SX_OK) return fail(rc, "split_tf32(B) launch failed");
      ++g_launches;
    }
    g.A = Ap; g.lda = p.a_ldp; g.a_plane_stride = p.M * p.a_ldp;
    g.B = Bp; g.ldb = p.b_ldp; g.b_plane_stride = p.N * p.b_ldp;
    g.bn = choose_kernel(p, d->tile_n, st->num_sms, 0, false).bn;
    if (opt.trace.load(std::memory_order_relaxed))
      fprintf(stderr, "[symplex_b200] gemm %lldx%lldx%lld batch %d f32 -> pre-split kernel, tile 128x%d\n", p.M, p.N, p.K,
              p.batch, g.bn);
    rc = launch_gemm_tf32x3(g, stream);
    if (rc == SX_ERR_EXEC) return fail(rc, "GEMM kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    if (rc != SX_OK) return rc;
    ++g_launches;
    return SX_OK;
  } else {
    const void* Ause = A;
    const void* Buse = B;
    long long lda = p.lda, ldb = p.ldb, a_bs = p.a_bs, b_bs = p.b_bs;
    if (p.a_prep) {
      if ((rc = need_scratch()) != SX_OK) return rc;
      rc = launch_repack_16(A, p.lda, p.a_bs, w + p.a_off, p.a_ldp, (int)p.M, (int)p.K, p.batch, stream);
      if (rc != SX_OK) return fail(rc, "repack(A) launch failed");
      ++g_launches;
      Ause = w + p.a_off; lda = p.a_ldp; a_bs = p.M * p.a_ldp;
    }
    if (p.b_prep) {
      if ((rc = need_scratch()) != SX_OK) return rc;
      if (!p.b_ready) {
        rc = launch_repack_16(B, p.ldb, p.b_bs, w + p.b_off, p.b_ldp, (int)p.b_rows, (int)p.b_cols, p.batch, stream);
        if (rc != SX_OK) return fail(rc, "repack(B) launch failed");
        ++g_launches;
      }
      Buse = w + p.b_off; ldb = p.b_ldp; b_bs = p.b_rows * p.b_ldp;
    }
    g.kind = 0;
    g.nseg = 1;
    g.a_planes = 1; g.b_planes = 1;
    g.za = p.batch; g.zb = p.batch;
    g.A = Ause; g.lda = lda; g.a_plane_stride = a_bs;
    g.B = Buse; g.ldb = ldb; g.b_plane_stride = b_bs;
  }
  if (n_peers > 7) return fail(SX_ERR_INVALID, "at most 7 peer destinations");
  g.bn = kc.bn;
  const int mode = kc.kind == KK_BF16_PAIR512 ? 2 : kc.kind == KK_BF16_PAIR256 ? 1 : 0;
  g.tma_store = opt.tma_store.load(std::memory_order_relaxed) != 0;
  if (n_peers > 0) {
    g.n_peers = n_peers;
    g.xchg = peers->xchg;
    g.my_rank = peers->my_rank;
    g.mc_C = peers->mc_C;
    g.flags = peers->flags;
    g.epoch = peers->epoch;
    g.xchg_counter = st->xchg_counter;
    for (int i = 0; i < n_peers; ++i) {
      g.peer_C[i] = peers->peer_C[i];
      g.peer_rank[i] = peers->peer_rank[i];
      g.peer_flags[i] = peers->peer_flags[i];
    }
  }
  if (mode == 2) g.bn = 512;
  if (kc.stream_k) {
    // The pool's mutex is held from here until the launch has been enqueued, so the flag words and the call number
    // have one user at a time; the pool's event orders the launches of different streams on the GPU.
    if ((rc = need_scratch()) != SX_OK) return rc;
    g.sk_ws = reinterpret_cast<float*>(w + sk_off);
    g.sk_flags = st->sk_flags;
    if (st->sk_epoch == 0x7fffffff) {  // the call number wraps: start over from cleared flags
      SX_CUDA(cudaDeviceSynchronize());
      SX_CUDA(cudaMemset(st->sk_flags, 0, stream_k_flag_words(st->num_sms) * sizeof(int)));
      st->sk_epoch = 0;
    }
    g.sk_epoch = ++st->sk_epoch;
  }
  if (opt.trace.load(std::memory_order_relaxed))
    fprintf(stderr, "[symplex_b200] gemm %lldx%lldx%lld batch %d bf16 -> %s%s, tile width %d, %d peer(s), exchange %d\n", p.M,
            p.N, p.K, p.batch, mode == 2 ? "512x256 CTA pairs" : mode == 1 ? "256x256 CTA pairs" : "single-CTA tiles",
            kc.stream_k ? " (stream-K)" : "", g.bn, n_peers, g.xchg);
  rc = mode != 0 ? launch_gemm_pair(g, stream) : launch_gemm_tc(g, stream);
  if (rc != SX_OK) {
    if (rc == SX_ERR_INVALID && strncmp(g_err, "cuTensorMap", 11) != 0)
      return fail(rc, "operands%s are not TMA compatible (16-byte alignment) or tile %d invalid",
                  n_peers > 0 ? " or peer buffers" : "", g.bn);
    if (rc == SX_ERR_EXEC) return fail(rc, "GEMM kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return rc;
  }
  ++g_launches;
  if (kc.stream_k) options().stream_k_launches.fetch_add(1, std::memory_order_relaxed);
  return SX_OK;
}

// ------------------------------------------------------------------ host-pointer path
struct HostCtx {
  cudaStream_t stream = nullptr;                  // compute (and, for small problems, everything)
  cudaStream_t h2d = nullptr, d2h = nullptr;      // copy streams of the row-chunked pipeline
  cudaEvent_t ev_in[64] = {}, ev_out[64] = {};    // chunk c: inputs landed / result ready
  bool pipeline_ready = false;
  void* buf[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // A, B, C, bias, residual, elementwise arena, GEMM scratch
  size_t cap[7] = {0, 0, 0, 0, 0, 0, 0};
  int dev = -1;
};
static thread_local HostCtx t_host;

static int host_buf(int i, size_t bytes, void** out) {
  HostCtx& h = t_host;
  if (bytes > h.cap[i]) {
    if (h.buf[i]) {
      SX_CUDA(cudaStreamSynchronize(h.stream));
      SX_CUDA(cudaFree(h.buf[i]));
      h.buf[i] = nullptr;
      h.cap[i] = 0;
    }
    const size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    SX_CUDA(cudaMalloc(&h.buf[i], want));
    h.cap[i] = want;
  }
  *out = h.buf[i];
  return SX_OK;
}

// The calling thread's streams: the compute stream always, the two copy streams and the per-chunk events of the
// chunked pipelines on request. A thread that moved to another device starts over with fresh buffers.
static int host_ctx(bool pipeline, HostCtx** out) {
  HostCtx& h = t_host;
  int dev = 0;
  SX_CUDA(cudaGetDevice(&dev));
  if (h.stream == nullptr || h.dev != dev) {
    SX_CUDA(cudaStreamCreateWithFlags(&h.stream, cudaStreamNonBlocking));
    h.dev = dev;
    h.pipeline_ready = false;
    for (int i = 0; i < 7; ++i) { h.buf[i] = nullptr; h.cap[i] = 0; }
  }
  if (pipeline && !h.pipeline_ready) {
    SX_CUDA(cudaStreamCreateWithFlags(&h.h2d, cudaStreamNonBlocking));
    SX_CUDA(cudaStreamCreateWithFlags(&h.d2h, cudaStreamNonBlocking));
    for (int i = 0; i < 64; ++i) {
      SX_CUDA(cudaEventCreateWithFlags(&h.ev_in[i], cudaEventDisableTiming));
      SX_CUDA(cudaEventCreateWithFlags(&h.ev_out[i], cudaEventDisableTiming));
    }
    h.pipeline_ready = true;
  }
  *out = &h;
  return SX_OK;
}

static int gemm_host(const symplex_gemm_desc* d, const void* A, const void* B, void* C, const float* bias,
                     const void* residual) {
  Plan p;
  int rc = make_plan(d, nullptr, nullptr, &p);  // device copies made here are always aligned
  if (rc != SX_OK) return rc;
  if (p.M == 0 || p.N == 0 || p.batch == 0) return SX_OK;
  if (A == nullptr || B == nullptr || C == nullptr) return fail(SX_ERR_INVALID, "null matrix pointer");
  DeviceState* st = nullptr;
  rc = device_state(&st);
  if (rc != SX_OK) return rc;
  HostCtx* hp = nullptr;
  if ((rc = host_ctx(false, &hp)) != SX_OK) return rc;
  HostCtx& h = *hp;
  const size_t in_elt = p.f32_in ? 4 : 2, out_elt = p.bf16_out ? 2 : 4;
  // Extent of each host operand including batch strides.
  const size_t a_bytes = ((size_t)(p.batch - 1) * p.a_bs + (size_t)(p.M - 1) * p.lda + p.K) * in_elt;
  const size_t b_bytes = ((size_t)(p.batch - 1) * p.b_bs + (size_t)(p.b_rows - 1) * p.ldb + p.b_cols) * in_elt;
  const size_t c_bytes = ((size_t)(p.batch - 1) * p.c_bs + (size_t)(p.M - 1) * p.ldc + p.N) * out_elt;
  if (p.K == 0) {
    return fail(SX_ERR_INVALID, "K == 0 is not supported");
  }
  void *dA, *dB, *dC, *dbias = nullptr, *dR = nullptr;
  if ((rc = host_buf(0, a_bytes, &dA)) != SX_OK) return rc;
  if ((rc = host_buf(1, b_bytes, &dB)) != SX_OK) return rc;
  if ((rc = host_buf(2, c_bytes, &dC)) != SX_OK) return rc;
  // Large single problems: split the rows of A / C into chunks and run a three-stream pipeline, so the
  // host -> device copy of chunk c+1, the GEMM of chunk c and the device -> host copy of chunk c-1 overlap.
  // Rows of C are independent, so the result is the one the single-shot path produces.
  {
    const size_t row_bytes = (size_t)p.K * in_elt + (size_t)p.N * out_elt;
    // bytes of A + C moved per chunk: 96 MB = ~2 ms of PCIe time, several waves of GEMM tiles
    const int64_t opt_mb = options().pipeline_mb.load(std::memory_order_relaxed);
    const size_t chunk_mb = opt_mb > 0 ? (size_t)opt_mb : 1;
    long long chunk_rows = (long long)((chunk_mb << 20) / row_bytes) / 512 * 512;
    if (chunk_rows < 2048) chunk_rows = 2048;
    if (chunk_rows * 64 < p.M) chunk_rows = ((p.M + 63) / 64 + 511) / 512 * 512;  // at most 64 chunks
    const long long nchunks = (p.M + chunk_rows - 1) / chunk_rows;
    const bool dense = p.lda == p.K && p.ldc == p.N;
    if (p.batch == 1 && dense && !residual && nchunks >= 3 && nchunks <= 64 &&
        options().pipeline.load(std::memory_order_relaxed) != 0) {
      if ((rc = host_ctx(true, &hp)) != SX_OK) return rc;
      Scratch scratch = Scratch::from_host_thread();  // the calling thread's own, never the shared pool
      SX_CUDA(cudaMemcpyAsync(dB, B, b_bytes, cudaMemcpyHostToDevice, h.h2d));
      if (bias) {
        if ((rc = host_buf(3, (size_t)p.N * 4, &dbias)) != SX_OK) return rc;
        SX_CUDA(cudaMemcpyAsync(dbias, bias, (size_t)p.N * 4, cudaMemcpyHostToDevice, h.h2d));
      }
      for (long long c = 0; c < nchunks; ++c) {
        const long long r0 = c * chunk_rows;
        const long long rows = (p.M - r0) < chunk_rows ? (p.M - r0) : chunk_rows;
        const uint8_t* hA = static_cast<const uint8_t*>(A) + (size_t)r0 * p.K * in_elt;
        uint8_t* dAc = static_cast<uint8_t*>(dA) + (size_t)r0 * p.K * in_elt;
        uint8_t* dCc = static_cast<uint8_t*>(dC) + (size_t)r0 * p.N * out_elt;
        SX_CUDA(cudaMemcpyAsync(dAc, hA, (size_t)rows * p.K * in_elt, cudaMemcpyHostToDevice, h.h2d));
        SX_CUDA(cudaEventRecord(h.ev_in[c], h.h2d));
        SX_CUDA(cudaStreamWaitEvent(h.stream, h.ev_in[c], 0));
        Plan pc = p;
        pc.M = rows;
        pc.a_bs = rows * p.lda;
        pc.c_bs = rows * p.ldc;
        pc.b_ready = c > 0;
        // this chunk's slice of the A scratch region (fp32 planes: 2 x rows x a_ldp floats; padded bf16: rows x a_ldp)
        pc.a_off = p.a_off + (size_t)r0 * p.a_ldp * (p.f32_in ? 8 : 2);
        rc = run_gemm(d, pc, dAc, dB, dCc, static_cast<const float*>(dbias), nullptr, scratch, st, h.stream);
        if (rc != SX_OK) {
          cudaStreamSynchronize(h.h2d);
          cudaStreamSynchronize(h.stream);
          cudaStreamSynchronize(h.d2h);
          return rc;
        }
        SX_CUDA(cudaEventRecord(h.ev_out[c], h.stream));
        SX_CUDA(cudaStreamWaitEvent(h.d2h, h.ev_out[c], 0));
        SX_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(C) + (size_t)r0 * p.N * out_elt, dCc, (size_t)rows * p.N * out_elt,
                                cudaMemcpyDeviceToHost, h.d2h));
      }
      int status = 0;
      SX_CUDA(cudaMemcpyAsync(&status, st->status, sizeof(int), cudaMemcpyDeviceToHost, h.d2h));
      SX_CUDA(cudaStreamSynchronize(h.d2h));
      SX_CUDA(cudaStreamSynchronize(h.stream));
      if (status != 0) {
        cudaMemsetAsync(st->status, 0, sizeof(int), h.stream);
        cudaStreamSynchronize(h.stream);
        return fail(SX_ERR_TIMEOUT, "device-side wait timed out (status %d); the output is not valid", status);
      }
      return SX_OK;
    }
  }
  SX_CUDA(cudaMemcpyAsync(dA, A, a_bytes, cudaMemcpyHostToDevice, h.stream));
  SX_CUDA(cudaMemcpyAsync(dB, B, b_bytes, cudaMemcpyHostToDevice, h.stream));
  if (bias) {
    if ((rc = host_buf(3, (size_t)p.N * 4, &dbias)) != SX_OK) return rc;
    SX_CUDA(cudaMemcpyAsync(dbias, bias, (size_t)p.N * 4, cudaMemcpyHostToDevice, h.stream));
  }
  if (residual) {
    if ((rc = host_buf(4, c_bytes, &dR)) != SX_OK) return rc;
    SX_CUDA(cudaMemcpyAsync(dR, residual, c_bytes, cudaMemcpyHostToDevice, h.stream));
  }
  if (p.ldc != p.N || (p.batch > 1 && p.c_bs != p.M * p.ldc)) {
    // Strided C: keep the bytes between rows that the kernel does not write.
    SX_CUDA(cudaMemcpyAsync(dC, C, c_bytes, cudaMemcpyHostToDevice, h.stream));
  }
  Scratch scratch = Scratch::from_host_thread();
  rc = run_gemm(d, p, dA, dB, dC, static_cast<const float*>(dbias), dR, scratch, st, h.stream);
  if (rc != SX_OK) return rc;
  SX_CUDA(cudaMemcpyAsync(C, dC, c_bytes, cudaMemcpyDeviceToHost, h.stream));
  int status = 0;
  SX_CUDA(cudaMemcpyAsync(&status, st->status, sizeof(int), cudaMemcpyDeviceToHost, h.stream));
  SX_CUDA(cudaStreamSynchronize(h.stream));
  if (status != 0) {
    cudaMemsetAsync(st->status, 0, sizeof(int), h.stream);
    cudaStreamSynchronize(h.stream);
    return fail(SX_ERR_TIMEOUT, "device-side wait timed out (status %d); the output is not valid", status);
  }
  return SX_OK;
}

static int64_t sgemm_host(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k) {
  if (m == 0 || n == 0 || k == 0) return 0;  // the reference returns before touching C
  if (m < 0 || n < 0 || k < 0) return fail(SX_ERR_INVALID, "negative dimension");
  symplex_gemm_desc d;
  symplex_b200_gemm_desc_init(&d, m, n, k, SYMPLEX_DT_F32, SYMPLEX_DT_F32);
  return gemm_host(&d, a, b, c, nullptr, nullptr);
}

// ------------------------------------------------------------------ fused elementwise programs
static_assert(sizeof(symplex_fused_op) == 8 && sizeof(FeSrcOp) == 8, "FusedOpDesc is 8 bytes");

static void* fe_reduce_scratch(DeviceState* st) {
  return st->fe_scratch + (st->fe_next.fetch_add(1) % FE_SCRATCH_SETS) * FE_REDUCE_SCRATCH_BYTES;
}

static int fe_device(const symplex_fused_op* ops, size_t n_ops, const void* const* inputs, size_t n_inputs,
                     const void* constants, size_t n_constants, int64_t n, int reduce_op, void* dst, double* result,
                     int elem_bytes, cudaStream_t stream) {
  if (n < 0) return fail(SX_ERR_INVALID, "negative element count");
  if (n == 0 || n_ops == 0) return SX_OK;  // the reference returns before touching anything
  auto prog = std::make_unique<FeProgram>();
  int rc = compile_fused_program(reinterpret_cast<const FeSrcOp*>(ops), n_ops, n_inputs, constants, n_constants,
                                 elem_bytes, prog.get());
  if (rc != SX_OK) return rc;
  DeviceState* st = nullptr;
  if ((rc = device_state(&st)) != SX_OK) return rc;
  void* red = reduce_op != FE_REDUCE_NONE ? fe_reduce_scratch(st) : nullptr;
  rc = launch_fused_elementwise(*prog, inputs, n, reduce_op, dst, result, red, st->status, st->num_sms, elem_bytes,
                                stream);
  if (rc == SX_OK) ++g_launches;
  return rc;
}

// Host arrays in, host array (or the reduced scalar) out. The element range is cut into chunks that run as a
// three-stream pipeline: copy-in of chunk c+1, the kernel on chunk c and copy-out of chunk c-1 overlap.
static int fe_host(const symplex_fused_op* ops, size_t n_ops, const void* const* inputs, size_t n_inputs,
                   const void* constants, size_t n_constants, size_t n, int reduce_op, void* dst, int elem_bytes,
                   double* value) {
  *value = 0.0;
  if (n == 0 || n_ops == 0) return SX_OK;
  const bool reduce = reduce_op != FE_REDUCE_NONE;
  if (reduce && (reduce_op < 0 || reduce_op > 2)) return fail(SX_ERR_INVALID, "reduce_op must be 0, 1, 2 or 255");
  if (!reduce && dst == nullptr) return fail(SX_ERR_INVALID, "null dst");
  auto prog = std::make_unique<FeProgram>();
  int rc = compile_fused_program(reinterpret_cast<const FeSrcOp*>(ops), n_ops, n_inputs, constants, n_constants,
                                 elem_bytes, prog.get());
  if (rc != SX_OK) return rc;
  for (int i = 0; i < prog->n_inputs; ++i)
    if (inputs == nullptr || inputs[prog->input_map[i]] == nullptr) return fail(SX_ERR_INVALID, "null input array");
  DeviceState* st = nullptr;
  if ((rc = device_state(&st)) != SX_OK) return rc;
  HostCtx* hp = nullptr;
  if ((rc = host_ctx(true, &hp)) != SX_OK) return rc;
  HostCtx& h = *hp;
  // Arena: one device array per used input, the output array, one double per chunk.
  const int ni = prog->n_inputs;
  const size_t eb = (size_t)elem_bytes;
  const size_t arr = align256(n * eb);
  void* arena = nullptr;
  if ((rc = host_buf(5, arr * (size_t)(ni + 1) + 64 * sizeof(double), &arena)) != SX_OK) return rc;
  char* base = static_cast<char*>(arena);
  double* d_res = reinterpret_cast<double*>(base + arr * (size_t)(ni + 1));
  size_t chunk = (size_t(32) << 20) / eb;  // elements per chunk: 32 MiB per array
  if (chunk * 64 < n) chunk = ((n + 63) / 64 + 4095) / 4096 * 4096;
  const int nchunks = (int)((n + chunk - 1) / chunk);
  // Device arrays are numbered like the compacted program inputs.
  auto dprog = std::make_unique<FeProgram>(*prog);
  for (int i = 0; i < ni; ++i) dprog->input_map[i] = i;
  const void* d_in[FE_MAX_INPUTS] = {};
  void* red = reduce ? fe_reduce_scratch(st) : nullptr;
  for (int c = 0; c < nchunks; ++c) {
    const size_t e0 = (size_t)c * chunk, cnt = (e0 + chunk <= n) ? chunk : n - e0;
    for (int i = 0; i < ni; ++i) {
      char* d = base + arr * (size_t)i + e0 * eb;
      SX_CUDA(cudaMemcpyAsync(d, static_cast<const char*>(inputs[prog->input_map[i]]) + e0 * eb, cnt * eb,
                              cudaMemcpyHostToDevice, h.h2d));
      d_in[i] = d;
    }
    SX_CUDA(cudaEventRecord(h.ev_in[c], h.h2d));
    SX_CUDA(cudaStreamWaitEvent(h.stream, h.ev_in[c], 0));
    char* d_dst = base + arr * (size_t)ni + e0 * eb;
    rc = launch_fused_elementwise(*dprog, d_in, (long long)cnt, reduce_op, d_dst, d_res + c, red, st->status,
                                  st->num_sms, elem_bytes, h.stream);
    if (rc != SX_OK) return rc;
    ++g_launches;
    if (!reduce) {
      SX_CUDA(cudaEventRecord(h.ev_out[c], h.stream));
      SX_CUDA(cudaStreamWaitEvent(h.d2h, h.ev_out[c], 0));
      SX_CUDA(cudaMemcpyAsync(static_cast<char*>(dst) + e0 * eb, d_dst, cnt * eb, cudaMemcpyDeviceToHost, h.d2h));
    }
  }
  double parts[64];
  int status = 0;
  if (reduce) SX_CUDA(cudaMemcpyAsync(parts, d_res, nchunks * sizeof(double), cudaMemcpyDeviceToHost, h.stream));
  SX_CUDA(cudaMemcpyAsync(&status, st->status, sizeof(int), cudaMemcpyDeviceToHost, h.stream));
  SX_CUDA(cudaStreamSynchronize(h.stream));
  SX_CUDA(cudaStreamSynchronize(h.d2h));
  if (status != 0) {
    SX_CUDA(cudaMemset(st->status, 0, sizeof(int)));
    return fail(SX_ERR_TIMEOUT, "device-side wait timed out (status %d)", status);
  }
  if (reduce) {
    double v = parts[0];
    for (int c = 1; c < nchunks; ++c)
      v = reduce_op == 0 ? v + parts[c] : reduce_op == 1 ? (parts[c] > v ? parts[c] : v) : (parts[c] < v ? parts[c] : v);
    *value = v;
  }
  return SX_OK;
}

// The void drop-ins have no return value to report a failure with (no device, out of memory, a device-side
// timeout). They make it impossible to miss instead: C is filled with NaN, and symplex_b200_last_error() holds the
// reason; after a successful call it reads "no error".
template <typename T>
static void void_abi_result(int64_t rc, T* C, size_t count) {
  if (rc == 0) {
    snprintf(g_err, sizeof(g_err), "no error");
    return;
  }
  if (C != nullptr)
    for (size_t i = 0; i < count; ++i) C[i] = std::numeric_limits<T>::quiet_NaN();
}

}  // namespace sx

// =================================================================== extern "C"
using namespace sx;

extern "C" {

void symplex_b200_gemm_desc_init(symplex_gemm_desc* d, int64_t M, int64_t N, int64_t K, int32_t in_dtype,
                                 int32_t out_dtype) {
  if (!d) return;
  memset(d, 0, sizeof(*d));
  d->M = M; d->N = N; d->K = K;
  d->batch = 1;
  d->in_dtype = in_dtype;
  d->out_dtype = out_dtype;
  d->b_layout = SYMPLEX_ROW_MAJOR;
  d->alpha = 1.0f;
  d->beta = 0.0f;
  d->activation = SYMPLEX_ACT_NONE;
}

size_t symplex_b200_gemm_workspace_bytes(const symplex_gemm_desc* d) {
  Plan p;
  // Pointer alignment is unknown here: size for the case where both bf16 operands need a padded copy.
  if (make_plan(d, reinterpret_cast<const void*>(1), reinterpret_cast<const void*>(1), &p) != SX_OK) return 0;
  return p.total;
}

int symplex_b200_gemm(const symplex_gemm_desc* d, const void* A, const void* B, void* C, const float* bias,
                      const void* residual, void* stream) {
  Plan p;
  int rc = make_plan(d, A, B, &p);
  if (rc != SX_OK) return rc;
  if (p.M == 0 || p.N == 0 || p.batch == 0) return SX_OK;
  if (!A || !B || !C) return fail(SX_ERR_INVALID, "null matrix pointer");
  DeviceState* st = nullptr;
  if ((rc = device_state(&st)) != SX_OK) return rc;
  Scratch scratch = Scratch::from_pool(st, static_cast<cudaStream_t>(stream));
  return run_gemm(d, p, A, B, C, bias, residual, scratch, st, static_cast<cudaStream_t>(stream));
}

int symplex_b200_gemm_peers(const symplex_gemm_desc* d, const void* A, const void* B, void* C, const float* bias,
                            const void* residual, const void* const* peer_C, int32_t n_peers, void* stream) {
  Plan p;
  int rc = make_plan(d, A, B, &p);
  if (rc != SX_OK) return rc;
  if (n_peers < 0 || (n_peers > 0 && peer_C == nullptr)) return fail(SX_ERR_INVALID, "bad peer list");
  if (p.M == 0 || p.N == 0 || p.batch == 0) return SX_OK;
  if (!A || !B || !C) return fail(SX_ERR_INVALID, "null matrix pointer");
  DeviceState* st = nullptr;
  if ((rc = device_state(&st)) != SX_OK) return rc;
  if (n_peers > 7) return fail(SX_ERR_INVALID, "at most 7 peer destinations");
  PeerArgs pa;
  pa.n_peers = n_peers;
  for (int i = 0; i < n_peers; ++i) pa.peer_C[i] = peer_C[i];
  Scratch scratch = Scratch::from_pool(st, static_cast<cudaStream_t>(stream));
  return run_gemm(d, p, A, B, C, bias, residual, scratch, st, static_cast<cudaStream_t>(stream), &pa);
}

int symplex_b200_sharded_gemm(const symplex_gemm_desc* d, const void* A_local, const void* B, const float* bias,
                              symplex_b200_comm* comm, int32_t exchange, void* stream) {
  if (d == nullptr || comm == nullptr) return fail(SX_ERR_INVALID, "null descriptor or communicator");
  const int world = comm->world, rank = comm->rank;
  if (world < 1 || world > SYMPLEX_B200_MAX_RANKS || rank < 0 || rank >= world)
    return fail(SX_ERR_INVALID, "bad communicator: rank %d of %d (at most %d ranks)", rank, world, SYMPLEX_B200_MAX_RANKS);
  if (d->batch != 1) return fail(SX_ERR_INVALID, "the sharded GEMM takes one problem (batch 1)");
  if (d->M % world != 0) return fail(SX_ERR_INVALID, "M = %lld rows do not split evenly over %d ranks", (long long)d->M, world);
  if (d->ldc != 0 && d->ldc != d->N) return fail(SX_ERR_INVALID, "the gathered C is dense: ldc must be N (or 0)");
  if (exchange < SYMPLEX_XCHG_AUTO || exchange > SYMPLEX_XCHG_EPILOGUE_TMA) return fail(SX_ERR_INVALID, "unknown exchange mode %d", exchange);
  if (comm->c_base[rank] == nullptr) return fail(SX_ERR_INVALID, "communicator has no local C buffer");
  symplex_gemm_desc dl = *d;  // this rank's share: rows [rank * M / world, (rank + 1) * M / world)
  dl.M = d->M / world;
  Plan p;
  int rc = make_plan(&dl, A_local, B, &p);
  if (rc != SX_OK) return rc;
  const size_t out_elt = p.bf16_out ? 2 : 4;
  const size_t row_off = (size_t)rank * (size_t)dl.M * (size_t)d->N * out_elt;
  uint8_t* C_local = static_cast<uint8_t*>(comm->c_base[rank]) + row_off;
  if (p.M == 0 || p.N == 0) return SX_OK;
  if (!A_local || !B) return fail(SX_ERR_INVALID, "null matrix pointer");
  DeviceState* st = nullptr;
  if ((rc = device_state(&st)) != SX_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Scratch scratch = Scratch::from_pool(st, s);
  if (world == 1) return run_gemm(&dl, p, A_local, B, C_local, bias, nullptr, scratch, st, s);
  if (p.f32_in) return fail(SX_ERR_INVALID, "the sharded GEMM takes bf16 inputs");
  PeerArgs pa;
  int mode = exchange;
  if (mode == SYMPLEX_XCHG_AUTO) mode = SYMPLEX_XCHG_UNICAST;
  if (mode == SYMPLEX_XCHG_MULTICAST && comm->c_multicast == nullptr)
    return fail(SX_ERR_INVALID, "exchange mode multicast needs comm->c_multicast (a multicast mapping of C)");
  pa.xchg = mode == SYMPLEX_XCHG_UNICAST ? XCHG_FORWARD : mode == SYMPLEX_XCHG_MULTICAST ? XCHG_MULTICAST : XCHG_EPILOGUE_TMA;
  pa.my_rank = rank;
  for (int r = 0; r < world; ++r) {
    if (r == rank) continue;
    if (comm->c_base[r] == nullptr) return fail(SX_ERR_INVALID, "communicator has no mapping of rank %d's C", r);
    pa.peer_C[pa.n_peers] = static_cast<uint8_t*>(comm->c_base[r]) + row_off;
    pa.peer_rank[pa.n_peers] = r;
    pa.peer_flags[pa.n_peers] = comm->flags[r];
    ++pa.n_peers;
  }
  if (pa.xchg != XCHG_EPILOGUE_TMA) {
    for (int r = 0; r < world; ++r)
      if (comm->flags[r] == nullptr) return fail(SX_ERR_INVALID, "communicator has no flag block for rank %d", r);
    pa.flags = comm->flags[rank];
    if (comm->c_multicast) pa.mc_C = static_cast<uint8_t*>(comm->c_multicast) + row_off;
    comm->epoch += 1;  // collective call number: every rank makes the same calls in the same order
    if ((uint32_t)comm->epoch == 0) comm->epoch += 1;  // flags start at 0: that value never names a call
    pa.epoch = (int)(uint32_t)comm->epoch;  // compared modulo 2^32 on the device
    if (comm->wait_limit_ms > 0) pa.wait_limit_ns = (unsigned long long)comm->wait_limit_ms * 1000000ull;
  }
  rc = run_gemm(&dl, p, A_local, B, C_local, bias, nullptr, scratch, st, s, &pa);
  if (rc != SX_OK && pa.xchg != XCHG_EPILOGUE_TMA) comm->epoch -= 1;  // nothing was launched: not a collective call
  return rc;
}

int symplex_b200_gemm_ws(const symplex_gemm_desc* d, const void* A, const void* B, void* C, const float* bias,
                         const void* residual, void* workspace, size_t workspace_bytes, void* stream) {
  Plan p;
  int rc = make_plan(d, A, B, &p);
  if (rc != SX_OK) return rc;
  if (p.M == 0 || p.N == 0 || p.batch == 0) return SX_OK;
  if (!A || !B || !C) return fail(SX_ERR_INVALID, "null matrix pointer");
  if (p.total > workspace_bytes || (p.total && workspace == nullptr))
    return fail(SX_ERR_INVALID, "workspace too small: need %zu bytes, got %zu", p.total, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) % 256) return fail(SX_ERR_INVALID, "workspace must be 256-byte aligned");
  DeviceState* st = nullptr;
  if ((rc = device_state(&st)) != SX_OK) return rc;
  Scratch scratch = Scratch::from_pointer(workspace);
  return run_gemm(d, p, A, B, C, bias, residual, scratch, st, static_cast<cudaStream_t>(stream));
}

int symplex_b200_sync_status(void* stream) {
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc != SX_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int status = 0;
  SX_CUDA(cudaMemcpyAsync(&status, st->status, sizeof(int), cudaMemcpyDeviceToHost, s));
  SX_CUDA(cudaStreamSynchronize(s));
  if (status != 0) {
    SX_CUDA(cudaMemsetAsync(st->status, 0, sizeof(int), s));
    SX_CUDA(cudaStreamSynchronize(s));
    return fail(SX_ERR_TIMEOUT, "device-side wait timed out (status %d)", status);
  }
  return SX_OK;
}

int symplex_b200_selftest_wait_timeout(const void* A, const void* B, void* C, int32_t limit_ms, void* stream) {
  if (!A || !B || !C) return fail(SX_ERR_INVALID, "null matrix pointer");
  if (limit_ms < 1 || limit_ms > 1000) return fail(SX_ERR_INVALID, "limit_ms must be in 1..1000");
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc != SX_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TcGemmArgs g{};
  g.kind = 0; g.out_bf16 = 1; g.b_mn = 1; g.bn = 64;
  g.M = 128; g.N = 64; g.K = 128;
  g.batch = 1; g.nseg = 1;
  g.a_planes = 1; g.b_planes = 1; g.za = 1; g.zb = 1;
  g.A = A; g.lda = 128; g.a_plane_stride = 128 * 128;
  g.B = B; g.ldb = 64; g.b_plane_stride = 128 * 64;
  g.C = C; g.ldc = 64; g.c_batch_stride = 128 * 64;
  g.alpha = 1.0f; g.beta = 0.0f; g.act = 0;
  g.status = st->status;
  g.num_sms = st->num_sms;
  g.wait_limit_ns = (unsigned long long)limit_ms * 1000000ull;
  g.fault_stop_early = 1;
  rc = launch_gemm_tc(g, s);
  if (rc != SX_OK) return fail(rc, "self-test launch failed: %s", cudaGetErrorString(cudaGetLastError()));
  ++g_launches;
  return symplex_b200_sync_status(stream);
}

int symplex_b200_set_option(const char* name, int64_t value) {
  std::atomic<int64_t>* v = option_by_name(name);
  if (v == nullptr) return fail(SX_ERR_INVALID, "unknown option '%s'", name ? name : "(null)");
  v->store(value);
  return SX_OK;
}

int64_t symplex_b200_get_option(const char* name) {
  std::atomic<int64_t>* v = option_by_name(name);
  return v ? v->load() : INT64_MIN;
}

const char* symplex_b200_last_error(void) { return g_err; }

int symplex_b200_gemm_host(const symplex_gemm_desc* d, const void* A, const void* B, void* C, const float* bias,
                           const void* residual) {
  return gemm_host(d, A, B, C, bias, residual);
}

int64_t symplex_cuda_matmul(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k) {
  return sgemm_host(a, b, c, m, n, k) == 0 ? 0 : -1;
}
int64_t symplex_parallel_matmul(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k) {
  return sgemm_host(a, b, c, m, n, k);
}
int64_t symplex_jit_parallel_matmul(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k) {
  return sgemm_host(a, b, c, m, n, k);
}
int64_t symplex_exec_matmul(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k) {
  return sgemm_host(a, b, c, m, n, k);
}
int64_t symplex_exec_fused_matmul_bias_relu(const float* a, const float* b, float* c, int64_t m, int64_t n,
                                            int64_t k, const float* bias) {
  if (m == 0 || n == 0) return 0;
  if (m < 0 || n < 0 || k <= 0) return fail(SX_ERR_INVALID, "bad dimension");
  symplex_gemm_desc d;
  symplex_b200_gemm_desc_init(&d, m, n, k, SYMPLEX_DT_F32, SYMPLEX_DT_F32);
  d.activation = SYMPLEX_ACT_RELU;
  return gemm_host(&d, a, b, c, bias, nullptr);
}

void symplex_matmul_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
  if (M > 0 && N > 0 && K == 0) {  // kernels/matmul.c zeroes C before accumulating
    memset(C, 0, (size_t)M * N * sizeof(float));
    snprintf(g_err, sizeof(g_err), "no error");
    return;
  }
  void_abi_result(sgemm_host(A, B, C, M, N, K), C, M > 0 && N > 0 ? (size_t)M * (size_t)N : 0);
}
void symplex_matmul_tiled_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
  symplex_matmul_f32(A, B, C, M, N, K);
}
void blas_sgemm(const float* a, const float* b, float* c, size_t m, size_t n, size_t k) {
  symplex_matmul_f32(a, b, c, (int64_t)m, (int64_t)n, (int64_t)k);
}
void cache_tiled_sgemm_thin(const float* a, const float* b, float* c, size_t m, size_t n, size_t k) {
  symplex_matmul_f32(a, b, c, (int64_t)m, (int64_t)n, (int64_t)k);
}

int symplex_b200_dgemm(const double* A, const double* B, double* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                       int64_t ldb, int64_t ldc, void* stream) {
  if (M < 0 || N < 0 || K < 0) return fail(SX_ERR_INVALID, "negative dimension");
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(SX_ERR_INVALID, "dimension exceeds 2^31-1");
  if (M == 0 || N == 0) return SX_OK;
  if (K == 0) return fail(SX_ERR_INVALID, "K == 0 is not supported by the device entry points");
  if (!A || !B || !C) return fail(SX_ERR_INVALID, "null matrix pointer");
  if (lda == 0) lda = K;
  if (ldb == 0) ldb = N;
  if (ldc == 0) ldc = N;
  if (lda < K || ldb < N || ldc < N) return fail(SX_ERR_INVALID, "leading dimension too small");
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc != SX_OK) return rc;
  rc = launch_dgemm(A, lda, B, ldb, C, ldc, (int)M, (int)N, (int)K, static_cast<cudaStream_t>(stream));
  if (rc == SX_ERR_EXEC) return fail(rc, "dgemm launch failed: %s", cudaGetErrorString(cudaGetLastError()));
  if (rc != SX_OK) return fail(rc, "dgemm: problem too large for one launch (more than 65535 x 64 rows)");
  ++g_launches;
  return SX_OK;
}

static int dgemm_host(const double* a, const double* b, double* c, size_t m, size_t n, size_t k) {
  if (m == 0 || n == 0) return SX_OK;
  if (k == 0) {  // the reference's loop nest leaves C = 0
    memset(c, 0, m * n * sizeof(double));
    return SX_OK;
  }
  if (!a || !b || !c) return fail(SX_ERR_INVALID, "null matrix pointer");
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc != SX_OK) return rc;
  HostCtx* hp = nullptr;
  if ((rc = host_ctx(false, &hp)) != SX_OK) return rc;
  void *dA, *dB, *dC;
  if ((rc = host_buf(0, m * k * 8, &dA)) != SX_OK) return rc;
  if ((rc = host_buf(1, k * n * 8, &dB)) != SX_OK) return rc;
  if ((rc = host_buf(2, m * n * 8, &dC)) != SX_OK) return rc;
  SX_CUDA(cudaMemcpyAsync(dA, a, m * k * 8, cudaMemcpyHostToDevice, hp->stream));
  SX_CUDA(cudaMemcpyAsync(dB, b, k * n * 8, cudaMemcpyHostToDevice, hp->stream));
  rc = symplex_b200_dgemm(static_cast<double*>(dA), static_cast<double*>(dB), static_cast<double*>(dC), (int64_t)m,
                          (int64_t)n, (int64_t)k, 0, 0, 0, hp->stream);
  if (rc != SX_OK) return rc;
  SX_CUDA(cudaMemcpyAsync(c, dC, m * n * 8, cudaMemcpyDeviceToHost, hp->stream));
  SX_CUDA(cudaStreamSynchronize(hp->stream));
  return SX_OK;
}

void blas_dgemm(const double* a, const double* b, double* c, size_t m, size_t n, size_t k) {
  void_abi_result(dgemm_host(a, b, c, m, n, k), c, m * n);
}
void cache_tiled_dgemm_thin(const double* a, const double* b, double* c, size_t m, size_t n, size_t k) {
  void_abi_result(dgemm_host(a, b, c, m, n, k), c, m * n);
}

int64_t symplex_b200_exec_tensor_matmul(const uint8_t* rec, size_t len, void* const* slots, size_t nslots) {
  // Wire format of Instr::TensorMatMul (rust-engine/src/types.rs:884-904): 0xA2, dst u16, lhs u16, rhs u16,
  // m u64, n u64, k u64, element_ty u8, lhs_layout u8, rhs_layout u8 - little endian, 34 bytes.
  if (rec == nullptr || len < 34) return fail(SX_ERR_INVALID, "TensorMatMul record needs 34 bytes, got %zu", len);
  if (rec[0] != 0xA2) return fail(SX_ERR_INVALID, "opcode 0x%02X is not TensorMatMul (0xA2)", rec[0]);
  auto u16 = [&](size_t o) { return (uint32_t)rec[o] | ((uint32_t)rec[o + 1] << 8); };
  auto u64 = [&](size_t o) {
    uint64_t v = 0;
    for (int i = 7; i >= 0; --i) v = (v << 8) | rec[o + i];
    return v;
  };
  const uint32_t dst = u16(1), lhs = u16(3), rhs = u16(5);
  const uint64_t m = u64(7), n = u64(15), k = u64(23);
  const int ety = rec[31], lhs_layout = rec[32], rhs_layout = rec[33];
  if (dst >= nslots || lhs >= nslots || rhs >= nslots || slots == nullptr)
    return fail(SX_ERR_INVALID, "slot index out of range (%u, %u, %u of %zu)", dst, lhs, rhs, nslots);
  if (ety != SYMPLEX_DT_F32 && ety != SYMPLEX_DT_BF16 && ety != SYMPLEX_DT_F64)
    return fail(SX_ERR_INVALID, "element type %d not supported on this path (F32 = 9, F64 = 10, BF16 = 11)", ety);
  if (lhs_layout != SYMPLEX_ROW_MAJOR) return fail(SX_ERR_INVALID, "lhs must be row-major");
  if (rhs_layout != SYMPLEX_ROW_MAJOR && rhs_layout != SYMPLEX_COL_MAJOR)
    return fail(SX_ERR_INVALID, "rhs layout byte %d is not a MatrixLayout", rhs_layout);
  if (m > 0x7fffffffULL || n > 0x7fffffffULL || k > 0x7fffffffULL) return fail(SX_ERR_INVALID, "dimension too large");
  if (m == 0 || n == 0 || k == 0) return 0;
  if (ety == SYMPLEX_DT_F64) {  // what the reference lowers to blas_dgemm / cache_tiled_dgemm_thin
    if (rhs_layout != SYMPLEX_ROW_MAJOR) return fail(SX_ERR_INVALID, "F64 records take a row-major rhs");
    return dgemm_host(static_cast<const double*>(slots[lhs]), static_cast<const double*>(slots[rhs]),
                      static_cast<double*>(slots[dst]), (size_t)m, (size_t)n, (size_t)k);
  }
  symplex_gemm_desc d;
  symplex_b200_gemm_desc_init(&d, (int64_t)m, (int64_t)n, (int64_t)k, ety, ety);
  d.b_layout = rhs_layout;
  return gemm_host(&d, slots[lhs], slots[rhs], slots[dst], nullptr, nullptr);
}

int symplex_b200_execute(const char* kernel_name, const symplex_kernel_args* a) {
  if (kernel_name == nullptr || a == nullptr) return fail(SX_ERR_INVALID, "null kernel name or arguments");
  const bool fused = strstr(kernel_name, "fused_matmul_bias_relu") != nullptr;
  if (!fused && strstr(kernel_name, "matmul") == nullptr)
    return fail(SX_ERR_INVALID, "kernel '%s' is not on this path (matmul, fused_matmul_bias_relu)", kernel_name);
  const int64_t need = fused ? 3 : 2;
  if (a->num_inputs < need || a->input_ptrs == nullptr)
    return fail(SX_ERR_INVALID, "kernel '%s' takes %lld inputs, got %lld", kernel_name, (long long)need,
                (long long)a->num_inputs);
  if (a->M < 0 || a->N < 0 || a->K < 0 || a->batch < 0) return fail(SX_ERR_INVALID, "negative dimension");
  if (a->M > 0x7fffffffLL || a->N > 0x7fffffffLL || a->K > 0x7fffffffLL || a->batch > 0x7fffffffLL)
    return fail(SX_ERR_INVALID, "dimension exceeds 2^31-1");
  if (a->M == 0 || a->N == 0 || a->K == 0 || a->batch == 0) return SX_OK;
  const int64_t want_in[3] = {a->batch * a->M * a->K * 4, a->batch * a->K * a->N * 4, a->N * 4};
  if (a->input_sizes != nullptr)
    for (int i = 0; i < need; ++i)
      if (a->input_sizes[i] < want_in[i])
        return fail(SX_ERR_INVALID, "input %d holds %lld bytes, the dimensions need %lld", i,
                    (long long)a->input_sizes[i], (long long)want_in[i]);
  if (a->data == nullptr || a->data_size < a->batch * a->M * a->N * 4)
    return fail(SX_ERR_INVALID, "output holds %lld bytes, the dimensions need %lld", (long long)a->data_size,
                (long long)(a->batch * a->M * a->N * 4));
  for (int i = 0; i < need; ++i)
    if (a->input_ptrs[i] == nullptr) return fail(SX_ERR_INVALID, "input %d is null", i);
  symplex_gemm_desc d;
  symplex_b200_gemm_desc_init(&d, a->M, a->N, a->K, SYMPLEX_DT_F32, SYMPLEX_DT_F32);
  d.batch = (int32_t)a->batch;
  if (fused) d.activation = SYMPLEX_ACT_RELU;
  return gemm_host(&d, a->input_ptrs[0], a->input_ptrs[1], a->data,
                   fused ? static_cast<const float*>(a->input_ptrs[2]) : nullptr, nullptr);
}

int symplex_cuda_available(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n < 1) {
    cudaGetLastError();
    return 0;
  }
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, 0) != cudaSuccess) return 0;
  return major == 10 ? 1 : 0;
}

int symplex_cuda_device_info(symplex_device_info* out) {
  if (!out) return fail(SX_ERR_INVALID, "null output");
  memset(out, 0, sizeof(*out));
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n < 1) {
    cudaGetLastError();
    return fail(SX_ERR_DRIVER, "no CUDA device: %s", e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  }
  cudaDeviceProp pr;
  SX_CUDA(cudaGetDeviceProperties(&pr, 0));
  strncpy(out->name, pr.name, sizeof(out->name) - 1);
  out->compute_capability_major = pr.major;
  out->compute_capability_minor = pr.minor;
  out->total_memory_bytes = pr.totalGlobalMem;
  out->num_sms = pr.multiProcessorCount;
  out->num_cuda_cores = pr.multiProcessorCount * 128;  // 4 x 32 fp32 lanes per SM on sm_100
  out->warp_size = pr.warpSize;
  out->max_threads_per_block = pr.maxThreadsPerBlock;
  out->max_shared_memory_per_block = (int32_t)pr.sharedMemPerBlock;
  int khz = 0;
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, 0);
  out->clock_mhz = khz / 1000;
  return SX_OK;
}

uint64_t symplex_b200_launch_count(void) { return g_launches.load(); }

int32_t symplex_b200_stream_k_items(int32_t pair, int32_t pairs, int32_t tiles, int32_t k_blocks, int32_t* items,
                                    int32_t cap, int32_t* contributors) {
  if (pairs <= 0 || pair < 0 || pair >= pairs || tiles <= 0 || k_blocks <= 0 || cap < 0) return -1;
  const int n = stream_k_work_items(pair, pairs, tiles, k_blocks, items, cap);
  if (contributors != nullptr && items != nullptr)
    for (int i = 0; i < n && i < cap; ++i)
      contributors[i] = items[4 * i + 3] == 2 ? stream_k_contributors(pair, pairs, tiles, k_blocks, items[4 * i]) : 0;
  return n;
}

int32_t symplex_b200_abi_sizes_ext(int32_t* out, int32_t n) {
  const int32_t sizes[] = {(int32_t)sizeof(symplex_gemm_desc),     (int32_t)sizeof(symplex_device_info),
                           (int32_t)sizeof(symplex_fused_op),      (int32_t)sizeof(symplex_b200_target),
                           (int32_t)sizeof(symplex_gemm_plan),     (int32_t)sizeof(symplex_b200_comm),
                           (int32_t)sizeof(symplex_shard_plan),    (int32_t)sizeof(symplex_generated_kernel),
                           (int32_t)sizeof(symplex_fusion_op),     (int32_t)sizeof(symplex_kernel_args)};
  const int32_t have = (int32_t)(sizeof(sizes) / sizeof(sizes[0]));
  for (int32_t i = 0; out != nullptr && i < n && i < have; ++i) out[i] = sizes[i];
  return have;
}

void symplex_b200_abi_sizes(int32_t out[5]) {
  if (!out) return;
  out[0] = (int32_t)sizeof(symplex_gemm_desc);
  out[1] = (int32_t)sizeof(symplex_device_info);
  out[2] = (int32_t)sizeof(symplex_fused_op);
  out[3] = (int32_t)sizeof(symplex_b200_target);
  out[4] = (int32_t)sizeof(symplex_gemm_plan);
}

int symplex_b200_fused_elementwise_plan(int n_inputs, int64_t n, int element_bytes, int num_sms,
                                        int32_t grid_dims[3], int32_t block_dims[3], int32_t* shared_mem_bytes) {
  if (n_inputs < 0 || n_inputs > FE_MAX_INPUTS || n <= 0 || (element_bytes != 4 && element_bytes != 8) || !grid_dims ||
      !block_dims || !shared_mem_bytes)
    return fail(SX_ERR_INVALID, "bad argument (0..16 input arrays, n > 0, 4- or 8-byte elements)");
  int g = 0, b = 0, sm = 0;
  describe_fused_elementwise(n_inputs, n, element_bytes, num_sms > 0 ? num_sms : 148, &g, &b, &sm);
  grid_dims[0] = g; grid_dims[1] = 1; grid_dims[2] = 1;
  block_dims[0] = b; block_dims[1] = 1; block_dims[2] = 1;
  *shared_mem_bytes = sm;
  return SX_OK;
}

int symplex_b200_hardware_target(symplex_b200_target* t) {
  if (!t) return fail(SX_ERR_INVALID, "null output");
  memset(t, 0, sizeof(*t));
  t->num_sms = 148;
  t->warp_size = 32;
  t->max_warps_per_sm = 64;
  t->max_threads_per_sm = 2048;
  t->shared_mem_bytes_per_sm = 228 * 1024;
  t->max_shared_mem_per_block = 227 * 1024;
  t->register_file_bytes_per_sm = 256 * 1024;
  t->tensor_memory_bytes_per_sm = 256 * 1024;
  t->max_registers_per_thread = 255;
  t->num_fp32_lanes_per_sm = 128;
  t->mma_m = 128;
  t->mma_n = 256;
  t->mma_k = 16;
  t->mma_pair_m = 256;
  strncpy(t->mma_dtype, "bf16", sizeof(t->mma_dtype) - 1);
  t->global_bw_gbps = 6552.0;       // STREAM-style copy measured on this library's target boards
  t->global_bw_nominal_gbps = 7700.0;
  t->bf16_dense_tflops = 1663.5;    // cuBLAS bf16, measured burst
  t->bf16_dense_tflops_sustained = 1396.0;
  t->bf16_dense_tflops_nominal = 2250.0;
  t->global_capacity_gb = 180.0;
  t->l2_cache_kb = 126 * 1024;
  t->nvlink_gbps_per_direction = 900.0;
  t->has_tma = 1;
  t->has_async_copy = 1;
  t->has_tensor_memory = 1;
  t->pipeline_stages = 4;
  int n = 0, dev = 0;
  if (cudaGetDeviceCount(&n) == cudaSuccess && n > 0 && cudaGetDevice(&dev) == cudaSuccess) {
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess && major == 10 &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) {
      t->num_sms = sms;
      t->from_device = 1;
    }
  } else {
    cudaGetLastError();
  }
  return SX_OK;
}

void symplex_b200_micro_kernel_config(uint8_t target, size_t element_bytes, size_t* out_tile_m, size_t* out_tile_n,
                                      size_t* out_tile_k, size_t* out_acc_regs, size_t* out_prefetch_dist) {
  size_t m, n, k, acc, pf;
  if (target == 3) {  // B200: one tcgen05.mma atom, accumulators counted in tensor-memory columns
    if (element_bytes == 2) {
      const KernelShape ks = describe_gemm_pair(2);
      m = 128, n = (size_t)ks.mma_n, k = (size_t)ks.mma_k, acc = (size_t)ks.tmem_cols, pf = (size_t)ks.stages - 1;
    } else {
      const KernelShape ks = describe_gemm_tf32x3(128);
      m = (size_t)ks.mma_m, n = (size_t)ks.mma_n, k = (size_t)ks.mma_k, acc = (size_t)ks.tmem_cols, pf = (size_t)ks.stages - 1;
    }
  } else if (target == 1) {  // EdgeDevice
    m = 4, n = 4, k = 8, acc = 4, pf = 1;
  } else if (target == 2) {  // TensorAccelerator
    m = 16, n = 16, k = 16, acc = 8, pf = 4;
  } else if (element_bytes == 2) {  // ServerX86, 16-bit
    m = 16, n = 16, k = 32, acc = 8, pf = 2;
  } else {  // ServerX86, fp32
    m = 8, n = 8, k = 8, acc = 16, pf = 1;
  }
  if (out_tile_m) *out_tile_m = m;
  if (out_tile_n) *out_tile_n = n;
  if (out_tile_k) *out_tile_k = k;
  if (out_acc_regs) *out_acc_regs = acc;
  if (out_prefetch_dist) *out_prefetch_dist = pf;
}

int symplex_b200_gemm_plan(const symplex_gemm_desc* d, int num_sms, symplex_gemm_plan* out) {
  if (!out) return fail(SX_ERR_INVALID, "null output");
  memset(out, 0, sizeof(*out));
  Plan p;
  int rc = make_plan(d, nullptr, nullptr, &p);
  if (rc != SX_OK) {
    strncpy(out->error, g_err, sizeof(out->error) - 1);
    return rc;
  }
  if (p.K == 0 || p.M == 0 || p.N == 0 || p.batch == 0) {
    rc = fail(SX_ERR_INVALID, "empty problem: nothing to plan");
    strncpy(out->error, g_err, sizeof(out->error) - 1);
    return rc;
  }
  if (num_sms <= 0) num_sms = 148;
  const KernelChoice kc = choose_kernel(p, d->tile_n, num_sms, 0, true, true);
  KernelShape ks;
  double eff;  // fraction of the tensor peak the variant sustains on large problems (measured)
  switch (kc.kind) {
    case KK_F32_FUSED:
      ks = f32_fused_tile_rows(p.M) == 64
               ? describe_gemm_f32_small()
               : describe_gemm_f32_fused(
                     f32_fused_split_k((long long)((p.M + 127) / 128) * ((p.N + 63) / 64) * p.batch, p.K, num_sms));
      eff = 0.45;
      break;
    case KK_F32_SPLIT: ks = describe_gemm_tf32x3(kc.bn); eff = 0.71; break;
    case KK_BF16_PAIR512: ks = describe_gemm_pair(2); eff = 0.90; break;
    case KK_BF16_PAIR256: ks = describe_gemm_pair(1); eff = 0.82; break;
    default: ks = describe_gemm_tc(kc.bn); eff = 0.70; break;
  }
  strncpy(out->kernel_name, ks.name, sizeof(out->kernel_name) - 1);
  out->tile_m = ks.tile_m; out->tile_n = ks.tile_n; out->tile_k = ks.tile_k;
  out->mma_m = ks.mma_m; out->mma_n = ks.mma_n; out->mma_k = ks.mma_k;
  out->cluster_size = ks.cluster;
  out->stages = ks.stages;
  out->shared_mem_bytes = ks.smem_bytes;
  out->tmem_columns = ks.tmem_cols;
  const long long mt = (p.M + ks.tile_m - 1) / ks.tile_m, nt = (p.N + ks.tile_n - 1) / ks.tile_n;
  out->tiles = mt * nt * p.batch;
  if (kc.kind == KK_F32_FUSED && f32_fused_tile_rows(p.M) == 64)
    out->tiles = nt * ((p.batch + 1) / 2);  // that kernel's unit of work holds two problems' 64 x 64 tiles
  const long long units = num_sms / ks.cluster;  // persistent: one CTA (or one cluster) per SM (group of SMs)
  const long long active = kc.stream_k ? units : out->tiles < units ? out->tiles : units;
  out->grid_dims[0] = (int32_t)(active * ks.cluster); out->grid_dims[1] = 1; out->grid_dims[2] = 1;
  out->block_dims[0] = ks.threads; out->block_dims[1] = 1; out->block_dims[2] = 1;
  out->prepass_launches = kc.kind == KK_F32_SPLIT ? 2 : (p.a_prep ? 1 : 0) + (p.b_prep ? 1 : 0);
  if (kc.kind == KK_F32_FUSED) out->prepass_launches = 0;
  out->workspace_bytes = kc.kind == KK_F32_FUSED ? 0 : p.total;
  const double in_elt = p.f32_in ? 4.0 : 2.0, out_elt = p.bf16_out ? 2.0 : 4.0;
  out->flops = 2.0 * (double)p.M * (double)p.N * (double)p.K * p.batch;
  out->bytes = ((double)p.M * p.K + (double)p.K * p.N) * in_elt * p.batch + (double)p.M * p.N * out_elt * p.batch;
  // Roofline estimate from the measured peaks: tensor time at the variant's sustained efficiency and at the
  // fraction of the machine the tiles can occupy (whole waves), HBM time for the algorithmic bytes (plus the
  // pre-pass's extra read and write of the operands), a fixed launch cost per kernel.
  const double peak = p.f32_in ? 1663.5e12 / 6.0 : 1663.5e12;
  const long long waves = (out->tiles + units - 1) / units;
  // Stream-K (the library's own scratch pool only, so not counted in workspace_bytes): every pair gets the same
  // number of k-blocks; the partial sums' trip through L2 costs about 4 %.
  const double occupancy = kc.stream_k ? 0.96 : (double)out->tiles / (double)(waves * units);
  const double t_tensor = out->flops / (peak * eff * occupancy);
  double hbm_bytes = out->bytes;
  if (kc.kind == KK_F32_SPLIT) hbm_bytes += 3.0 * ((double)p.M * p.K + (double)p.K * p.N) * 4.0 * p.batch;
  const double t_hbm = hbm_bytes / (kc.kind == KK_F32_FUSED ? 0.64 * 6552e9 : 6552e9);  // fused: measured streaming rate
  // The in-kernel-split fp32 kernel serves small problems, where filling and draining its pipeline (first
  // loads, conversion, MMA completion, accumulator drain, teardown: ~7 us measured) is most of the run time.
  const double t = (t_tensor > t_hbm ? t_tensor : t_hbm) + 4e-6 * (1 + out->prepass_launches) +
                   (kc.kind == KK_F32_FUSED ? 7e-6 : 0.0);
  out->estimated_latency_ns = t * 1e9;
  out->estimated_tflops = out->flops / t / 1e12;
  out->bound = t_tensor >= t_hbm ? 0 : 1;
  // "Naive" = the one-thread-per-output scalar-FMA kernel the reference's PTX generator describes
  // (rust-engine/src/cuda_backend.rs:300-504): two shared-memory loads per FMA, i.e. at most
  // 148 SMs x 128 B/clk / 8 B x 2 flop x 1.9 GHz = 9 TFLOP/s.
  out->speedup_vs_naive = (out->flops / 9e12 + 4e-6) / t;
  out->valid = 1;
  return SX_OK;
}

int symplex_b200_fused_elementwise_f32(const symplex_fused_op* ops, size_t n_ops, const float* const* inputs,
                                       size_t n_inputs, const float* constants, size_t n_constants, int64_t n,
                                       int reduce_op, float* dst, double* result, void* stream) {
  return fe_device(ops, n_ops, reinterpret_cast<const void* const*>(inputs), n_inputs, constants, n_constants, n,
                   reduce_op, dst, result, 4, static_cast<cudaStream_t>(stream));
}
int symplex_b200_fused_elementwise_f64(const symplex_fused_op* ops, size_t n_ops, const double* const* inputs,
                                       size_t n_inputs, const double* constants, size_t n_constants, int64_t n,
                                       int reduce_op, double* dst, double* result, void* stream) {
  return fe_device(ops, n_ops, reinterpret_cast<const void* const*>(inputs), n_inputs, constants, n_constants, n,
                   reduce_op, dst, result, 8, static_cast<cudaStream_t>(stream));
}

static double fe_host_value(const symplex_fused_op* ops, size_t n_ops, const void* const* inputs, size_t n_inputs,
                            const void* constants, size_t n_constants, size_t n, int reduce_op, void* dst,
                            int elem_bytes) {
  double v = 0.0;
  const int rc = fe_host(ops, n_ops, inputs, n_inputs, constants, n_constants, n, reduce_op, dst, elem_bytes, &v);
  if (rc != SX_OK) return __builtin_nan("");
  snprintf(g_err, sizeof(g_err), "no error");  // lets a caller tell a computed NaN from a failure
  return v;
}
double symplex_simd_fused_elementwise_f32(const symplex_fused_op* ops, size_t n_ops, const float* const* input_ptrs,
                                          size_t n_inputs, const float* constants, size_t n_constants, size_t n,
                                          uint8_t reduce_op, float* dst_ptr) {
  return fe_host_value(ops, n_ops, reinterpret_cast<const void* const*>(input_ptrs), n_inputs, constants, n_constants,
                       n, reduce_op, dst_ptr, 4);
}
double symplex_simd_fused_elementwise_f64(const symplex_fused_op* ops, size_t n_ops, const double* const* input_ptrs,
                                          size_t n_inputs, const double* constants, size_t n_constants, size_t n,
                                          uint8_t reduce_op, double* dst_ptr) {
  return fe_host_value(ops, n_ops, reinterpret_cast<const void* const*>(input_ptrs), n_inputs, constants, n_constants,
                       n, reduce_op, dst_ptr, 8);
}

int64_t symplex_cuda_elementwise(const float* a, const float* b, float* dst, int64_t n, int op) {
  if (n == 0) return 0;
  if (op < 0 || op > 5) return -2;  // unknown op, like cuda_elementwise_raw
  if (n < 0 || !a || !b || !dst) {
    fail(SX_ERR_INVALID, "bad argument");
    return -1;
  }
  const symplex_fused_op prog = {(uint8_t)op, 0, 0, 0, 0, 1};
  const void* in[2] = {a, b};
  double v = 0.0;
  return fe_host(&prog, 1, in, 2, nullptr, 0, (size_t)n, FE_REDUCE_NONE, dst, 4, &v) == SX_OK ? 0 : -1;
}

int symplex_b200_fused_program_info(const symplex_fused_op* ops, size_t n_ops, size_t n_inputs, int* n_slots,
                                    int* n_inputs_used) {
  auto prog = std::make_unique<FeProgram>();
  static const float zeros[1] = {0.0f};
  const int rc = compile_fused_program(reinterpret_cast<const FeSrcOp*>(ops), n_ops, n_inputs, zeros, 0, 4, prog.get());
  if (rc != SX_OK) return rc;
  if (n_slots) *n_slots = prog->n_slots;
  if (n_inputs_used) *n_inputs_used = prog->n_inputs;
  return SX_OK;
}

}  // extern "C"
