// fp32-accurate GEMM on the tcgen05 tensor cores: the 3xTF32 scheme with round-to-nearest accumulation.
//
// Each fp32 operand x is held as two tf32 planes, hi = tf32(x) and lo = tf32(x - hi) (prep_kernels.cu).
// The product is  A.B ~= Ahi.Bhi + Ahi.Blo + Alo.Bhi  (the dropped Alo.Blo term is ~2^-22 relative).
//
// The tensor core adds into its fp32 accumulator with truncation, so a single long accumulation
// drifts by about (number of MMA steps) x 2^-25 - measurably above 1e-5 at K = 4096. This kernel
// therefore keeps every in-tensor-core accumulation short or small:
//   * Ahi.Bhi is accumulated in TMEM only over a chunk of CHUNK_KB k-blocks (K = 128), then drained by
//     the epilogue warps into fp32 registers with ordinary round-to-nearest adds;
//   * the two correction products go to a separate TMEM accumulator whose magnitude is 2^-11 of the
//     result, so its truncation error is negligible; it is added once at the end of the tile.
//
//   warp 0      TMA producer (one elected thread): per k-block one box of {hi,lo} for A and one for B
//   warp 1      MMA issuer (one elected thread): 3 tcgen05.mma.kind::tf32 per 8-wide k step
//   warps 2..5  accumulate chunk partials from TMEM, then alpha / beta / bias / activation and stores
//
// Serves the fp32 entry points of the reference's path: symplex_matmul_f32, jit_parallel_matmul,
// cuda_matmul, the fused matmul+bias+ReLU kernel (rust-engine/src/x86_emitter.rs:437-770).
#include <cuda_bf16.h>

#include "epilogue.cuh"
#include "gemm_params.h"
#include "host_api.h"
#include "sm100_ptx.cuh"

namespace sx {

template <int kBN>
struct X3Cfg {
  static constexpr int BM = 128;
  static constexpr int BN = kBN;
  static constexpr int BK = 32;      // 128 bytes of fp32
  static constexpr int UMMA_K = 8;
  static constexpr int CHUNK_KB = 4;  // k-blocks accumulated inside the tensor core before a drain
  static constexpr int A_PLANE = BM * 128;
  static constexpr int B_PLANE = BN * 128;
  static constexpr int STAGE_BYTES = 2 * A_PLANE + 2 * B_PLANE;
  static constexpr int STAGES = (196 * 1024) / STAGE_BYTES;
  static constexpr int TMEM_COLS = 4 * BN;  // main[2] + corr[2]
  static constexpr int DYN_SMEM = STAGES * STAGE_BYTES + 1024;
  static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM columns");
};

// Tile order: bands of group_m tile rows, column-major inside a band, so the tiles that run at the same time share
// a band of A planes (group_m x 128 rows) and a sliding window of B planes that together fit in L2; walking all
// tile rows of a column first (the whole of A's planes per column) re-streamed A from DRAM for every few columns.
__device__ __forceinline__ void x3_tile(const GemmParams& p, int r, int BM, int BN, int& m0, int& n0) {
  const int band = p.group_m * p.n_tiles;
  const int g = r / band;
  const int first_m = g * p.group_m;
  const int gsz = min(p.m_tiles - first_m, p.group_m);
  const int in_band = r - g * band;
  m0 = (first_m + in_band % gsz) * BM;
  n0 = (in_band / gsz) * BN;
}

template <typename OutT, int kBN>
__global__ void __launch_bounds__(192, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const GemmParams p) {
  using Cfg = X3Cfg<kBN>;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES, CH = Cfg::CHUNK_KB;

  extern __shared__ uint8_t dyn_smem[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES];
  __shared__ uint64_t main_full[2], main_empty[2], corr_full[2], corr_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&main_full[a], 1);
      mbar_init(&main_empty[a], 4);
      mbar_init(&corr_full[a], 1);
      mbar_init(&corr_empty[a], 4);
    }
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(&tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_launch_dependents();  // the next kernel in the stream may set itself up on SMs this grid leaves
  pdl_wait_prior_grids();   // the kernel before this one has completed: its outputs may be this one's operands

  const int per = p.m_tiles * p.n_tiles;
  const int total_tiles = p.batch * per;
  const int nkb = (p.K + BK - 1) / BK;
  const int nchunks = (nkb + CH - 1) / CH;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0, armed = 0, armed_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const int z = t / per, r = t - z * per;
        int m0, n0;
        x3_tile(p, r, BM, BN, m0, n0);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, &abort_flag)) { ok = false; break; }
          uint8_t* sa = tiles + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + 2 * Cfg::A_PLANE;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          armed |= 1u << stage;
          armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
          tma_load_3d(sa, &tmA, &full_bar[stage], kb * BK, m0, z * 2);  // box depth 2: hi plane, lo plane
          tma_load_3d(sb, &tmB, &full_bar[stage], kb * BK, n0, z * 2);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        for (int s = 0; s < STAGES; ++s) {
          if (!(armed & (1u << s))) continue;
          while (!mbar_try_wait(&full_bar[s], (armed_phase >> s) & 1u)) {
            if (globaltimer_ns() - t0 > 2000000ull) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(2, false, false, BM, BN);
      constexpr uint64_t dhi = make_smem_desc_hi(16, 1024);
      int stage = 0;
      uint32_t phase = 0;
      int macc = 0, cacc = 0;
      uint32_t mphase = 0, cphase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        if (!mbar_wait(&corr_empty[cacc], cphase ^ 1, &abort_flag)) break;
        const uint32_t d_corr = tmem_base + 2 * BN + cacc * BN;
        int kb = 0;
        for (int ch = 0; ok && ch < nchunks; ++ch) {
          if (!mbar_wait(&main_empty[macc], mphase ^ 1, &abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t d_main = tmem_base + macc * BN;
          const int kb_end = min(kb + CH, nkb);
          for (int kc = 0; kb < kb_end; ++kb, ++kc) {
            if (!mbar_wait(&full_bar[stage], phase, &abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t a_hi = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
            const uint32_t a_lo = a_hi + Cfg::A_PLANE;
            const uint32_t b_hi = a_hi + 2 * Cfg::A_PLANE;
            const uint32_t b_lo = b_hi + Cfg::B_PLANE;
#pragma unroll
            for (int k = 0; k < BK / Cfg::UMMA_K; ++k) {
              const uint32_t o = k * 32;
              umma<1, 1>(d_main, smem_desc(dhi, a_hi + o), smem_desc(dhi, b_hi + o), idesc, (kc | k) != 0 ? 1u : 0u);
              umma<1, 1>(d_corr, smem_desc(dhi, a_hi + o), smem_desc(dhi, b_lo + o), idesc, (kb | k) != 0 ? 1u : 0u);
              umma<1, 1>(d_corr, smem_desc(dhi, a_lo + o), smem_desc(dhi, b_hi + o), idesc, 1u);
            }
            umma_commit(&empty_bar[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          umma_commit(&main_full[macc]);
          if (++macc == 2) { macc = 0; mphase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&corr_full[cacc]);
        if (++cacc == 2) { cacc = 0; cphase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ accumulate + epilogue (warps 2..5)
    const int q = warp & 3;
    const EpilogueCtx<OutT> ep(p);
    const uint32_t lane_base = uint32_t(q * 32) << 16;
    int macc = 0, cacc = 0;
    uint32_t mphase = 0, cphase = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      const int z = t / per, r = t - z * per;
      int m0, n0;
      x3_tile(p, r, BM, BN, m0, n0);
      float sum[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) sum[j] = 0.0f;
      for (int ch = 0; ch < nchunks; ++ch) {
        if (!mbar_wait(&main_full[macc], mphase, &abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t rr[32];
          tmem_ld_32x32(tmem_base + lane_base + macc * BN + c * 32, rr);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) sum[c * 32 + j] += __uint_as_float(rr[j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&main_empty[macc]);
        if (++macc == 2) { macc = 0; mphase ^= 1; }
      }
      if (!ok) break;
      if (!mbar_wait(&corr_full[cacc], cphase, &abort_flag)) break;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32(tmem_base + lane_base + 2 * BN + cacc * BN + c * 32, rr);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[c * 32 + j] += __uint_as_float(rr[j]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&corr_empty[cacc]);
      if (++cacc == 2) { cacc = 0; cphase ^= 1; }

      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const long long row_off = (long long)z * p.c_batch_stride + (long long)row * p.ldc;
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = sum[c * 32 + j];
        ep.template strip<false>(v, row_ok, row_off, col0);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && abort_flag != 0 && p.status != nullptr) atomicExch(p.status, int(ST_WAIT_TIMEOUT));
}

// ------------------------------------------------------------------ host side
namespace {

template <typename OutT, int kBN>
int launch_x3(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid, cudaStream_t stream) {
  using Cfg = X3Cfg<kBN>;
  auto kern = gemm_tf32x3_kernel<OutT, kBN>;
  SX_ENSURE_DYN_SMEM(kern, Cfg::DYN_SMEM);
  return launch_kernel_ex(kern, (unsigned)grid, 192u, Cfg::DYN_SMEM, stream, 1, pdl_enabled(), tmA, tmB, p) == cudaSuccess
             ? SX_OK
             : SX_ERR_EXEC;
}

}  // namespace

// A planes: [batch][2][M][lda] fp32, B planes: [batch][2][N][ldb] fp32 (both K contiguous).
int launch_gemm_tf32x3(const TcGemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) return SX_ERR_INVALID;
  if (a.lda % 4 || a.ldb % 4 || a.a_plane_stride % 4 || a.b_plane_stride % 4) return SX_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(a.A) % 16 || reinterpret_cast<uintptr_t>(a.B) % 16) return SX_ERR_INVALID;
  const int bn = a.bn;
  if (bn != 128 && bn != 64) return SX_ERR_INVALID;

  CUtensorMap tmA, tmB;
  {
    uint64_t dims[3] = {(uint64_t)a.K, (uint64_t)a.M, (uint64_t)(2 * a.batch)};
    uint64_t strides[2] = {(uint64_t)a.lda * 4, (uint64_t)a.a_plane_stride * 4};
    uint32_t box[3] = {32u, 128u, 2u};
    int rc = encode_tensor_map_3d(&tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.A, dims, strides, box);
    if (rc != SX_OK) return rc;
  }
  {
    uint64_t dims[3] = {(uint64_t)a.K, (uint64_t)a.N, (uint64_t)(2 * a.batch)};
    uint64_t strides[2] = {(uint64_t)a.ldb * 4, (uint64_t)a.b_plane_stride * 4};
    uint32_t box[3] = {32u, (uint32_t)bn, 2u};
    int rc = encode_tensor_map_3d(&tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.B, dims, strides, box);
    if (rc != SX_OK) return rc;
  }

  GemmParams p{};
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.batch = a.batch;
  p.C = a.C; p.ldc = a.ldc; p.c_batch_stride = a.c_batch_stride;
  p.bias = a.bias; p.residual = a.residual;
  p.alpha = a.alpha; p.beta = a.beta; p.act = a.act;
  p.status = a.status;
  p.m_tiles = (int)((a.M + 127) / 128);
  p.n_tiles = (int)((a.N + bn - 1) / bn);
  p.group_m = a.group_m > 0 ? a.group_m : 8;
  const long long total = (long long)p.batch * p.m_tiles * p.n_tiles;
  const int grid = (int)(total < a.num_sms ? total : a.num_sms);
  if (a.out_bf16) {
    return bn == 128 ? launch_x3<__nv_bfloat16, 128>(tmA, tmB, p, grid, stream)
                     : launch_x3<__nv_bfloat16, 64>(tmA, tmB, p, grid, stream);
  }
  return bn == 128 ? launch_x3<float, 128>(tmA, tmB, p, grid, stream) : launch_x3<float, 64>(tmA, tmB, p, grid, stream);
}


KernelShape describe_gemm_tf32x3(int bn) {
  auto mk = [](auto cfg) {
    using C = decltype(cfg);
    return KernelShape{"gemm_tf32x3_kernel", C::BM, C::BN, C::BK, C::BM, C::BN, C::UMMA_K, 192, 1, C::STAGES, C::DYN_SMEM, C::TMEM_COLS};
  };
  return bn == 128 ? mk(X3Cfg<128>{}) : mk(X3Cfg<64>{});
}

}  // namespace sx
