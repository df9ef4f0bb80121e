// Persistent, warp-specialised tcgen05 GEMM for sm_100a (one CTA per SM, 128 x BN output tiles).
//
//   warp 0      TMA producer: streams 128B-swizzled A / B tiles into a ring of shared-memory stages
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (accumulators live in TMEM)
//   warps 2..5  epilogue: tcgen05.ld -> registers -> alpha / beta / bias / activation -> global stores
//
// TMEM holds two accumulators, so the epilogue of tile t overlaps the main loop of tile t+1.
// A launch is a flat list of (batch z, m-tile, n-tile) work items walked with a fixed stride by every
// CTA; the k loop runs over `nseg` operand-plane pairs, which is how the 3xTF32 product
// (hi*hi + hi*lo + lo*hi) and the plain bf16 product share one main loop.
//
// Replaces the matmul lowering of the reference's PTX text generator
// (rust-engine/src/cuda_backend.rs:300-504, gen_matmul) and its host wrapper (:1344-1385).
#include <cuda_bf16.h>

#include "epilogue.cuh"
#include "gemm_params.h"
#include "host_api.h"
#include "sm100_ptx.cuh"

namespace sx {

template <int kBN, int kKind>
struct TileCfg {
  static constexpr int BM = 128;
  static constexpr int BN = kBN;
  static constexpr int ELT = kKind == 0 ? 2 : 4;   // bytes per input element
  static constexpr int BK = 128 / ELT;             // one 128-byte swizzle row of K per stage
  static constexpr int UMMA_K = 32 / ELT;          // K per tcgen05.mma
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = (196 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int B_CHUNK = 128 / ELT;        // MN elements per swizzle row when B is MN-major
  static constexpr int B_CHUNKS = BN / B_CHUNK;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int DYN_SMEM = STAGES * STAGE_BYTES + 1024;
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns: power of two <= 512");
};

struct TileCoord {
  int z, m0, n0;
};

template <int BM, int BN>
__device__ __forceinline__ TileCoord tile_coord(const GemmParams& p, int t) {
  const int per = p.m_tiles * p.n_tiles;
  const int z = t / per;
  const int r = t - z * per;
  const int band = p.group_m * p.n_tiles;      // tiles in one band of group_m tile rows
  const int g = r / band;
  const int first_m = g * p.group_m;
  const int gsz = min(p.m_tiles - first_m, p.group_m);
  const int in_band = r - g * band;
  TileCoord c;
  c.z = z;
  c.m0 = (first_m + in_band % gsz) * BM;
  c.n0 = (in_band / gsz) * BN;
  return c;
}

template <typename OutT, int kBN, bool kBmn, int kKind>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const GemmParams p) {
  using Cfg = TileCfg<kBN, kKind>;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES;

  extern __shared__ uint8_t dyn_smem[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
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
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
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

  const int total_tiles = p.batch * p.m_tiles * p.n_tiles;
  const int nkb = (p.K + BK - 1) / BK;
  const int iters = nkb * p.nseg;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0, armed_phase = 0;  // stages whose loads may still be in flight
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const TileCoord tc = tile_coord<BM, BN>(p, t);
        for (int it = 0; it < iters; ++it) {
          const int seg = it / nkb;
          const int kb = it - seg * nkb;
          // Self-test of the unwinding (symplex_b200_selftest_wait_timeout): the last k-block is never loaded, so
          // the MMA thread's wait for it runs out; nothing asynchronous is left in flight by this thread.
          if (p.fault_stop_early && it == iters - 1) { ok = false; break; }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, &abort_flag, p.wait_limit_ns)) { ok = false; break; }
          uint8_t* sa = tiles + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          armed |= 1u << stage;
          armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
          tma_load_3d(sa, &tmA, &full_bar[stage], kb * BK, tc.m0, tc.z * p.a_planes + p.a_plane[seg]);
          const int zb = tc.z * p.b_planes + p.b_plane[seg];
          if constexpr (kBmn) {
#pragma unroll
            for (int c = 0; c < Cfg::B_CHUNKS; ++c)
              tma_load_3d(sb + c * (BK * 128), &tmB, &full_bar[stage], tc.n0 + c * Cfg::B_CHUNK, kb * BK, zb);
          } else {
            tma_load_3d(sb, &tmB, &full_bar[stage], kb * BK, tc.n0, zb);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Unwinding: give copies that were already issued a bounded time to land.
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
      constexpr uint32_t idesc = make_idesc(kKind == 0 ? 1 : 2, false, kBmn, BM, BN);
      constexpr uint64_t a_hi = make_smem_desc_hi(16, 1024);
      // B held MN-major: shared-memory rows are 128 B of N; 8 K-rows form a 1024-B swizzle atom (SBO);
      // successive 128-B column chunks of the tile are separate TMA boxes of BK K-rows each (LBO).
      constexpr uint64_t b_hi = kBmn ? make_smem_desc_hi(BK * 128, 1024) : make_smem_desc_hi(16, 1024);
      constexpr uint32_t b_kstep = kBmn ? Cfg::UMMA_K * 128 : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, &abort_flag, p.wait_limit_ns)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int it = 0; it < iters; ++it) {
          if (!mbar_wait(&full_bar[stage], phase, &abort_flag, p.wait_limit_ns)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / Cfg::UMMA_K; ++k) {
            umma<1, kKind>(d_tmem, smem_desc(a_hi, a_addr + k * 32), smem_desc(b_hi, b_addr + k * b_kstep), idesc,
                           (it | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const EpilogueCtx<OutT> ep(p);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const TileCoord tc = tile_coord<BM, BN>(p, t);
      if (!mbar_wait(&acc_full[acc], acc_phase, &abort_flag, p.wait_limit_ns)) break;
      tc_fence_after_sync();
      const int row = tc.m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const long long row_off = (long long)tc.z * p.c_batch_stride + (long long)row * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        const int col0 = tc.n0 + c * 32;
        if (col0 >= p.N) continue;  // uniform across the warp
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        ep.template strip<true>(v, row_ok, row_off, col0);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
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

template <typename OutT, int kBN, bool kBmn, int kKind>
int launch_one(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid, cudaStream_t stream) {
  using Cfg = TileCfg<kBN, kKind>;
  auto kern = gemm_tc_kernel<OutT, kBN, kBmn, kKind>;
  SX_ENSURE_DYN_SMEM(kern, Cfg::DYN_SMEM);
  return launch_kernel_ex(kern, (unsigned)grid, 192u, Cfg::DYN_SMEM, stream, 1, pdl_enabled(), tmA, tmB, p) == cudaSuccess
             ? SX_OK
             : SX_ERR_EXEC;
}

template <typename OutT, bool kBmn, int kKind>
int launch_bn(int bn, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid,
              cudaStream_t stream) {
  switch (bn) {
    case 256: return launch_one<OutT, 256, kBmn, kKind>(tmA, tmB, p, grid, stream);
    case 128: return launch_one<OutT, 128, kBmn, kKind>(tmA, tmB, p, grid, stream);
    case 64: return launch_one<OutT, 64, kBmn, kKind>(tmA, tmB, p, grid, stream);
    default: return SX_ERR_INVALID;
  }
}

}  // namespace

int pick_bn(long long M, long long N, int batch, int num_sms, int forced) {
  if (forced == 256 || forced == 128 || forced == 64) return forced;
  const long long mt = (M + 127) / 128;
  for (int bn : {256, 128}) {
    if (N < bn) continue;
    if (mt * ((N + bn - 1) / bn) * batch >= num_sms) return bn;
  }
  return 64;
}

int launch_gemm_tc(const TcGemmArgs& a, cudaStream_t stream) {
  const int kind = a.kind;
  const int elt = kind == 0 ? 2 : 4;
  const int bk = 128 / elt;
  const int bn = a.bn;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) return SX_ERR_INVALID;
  if ((a.lda * elt) % 16 || (a.ldb * elt) % 16 || (a.a_plane_stride * elt) % 16 || (a.b_plane_stride * elt) % 16)
    return SX_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(a.A) % 16 || reinterpret_cast<uintptr_t>(a.B) % 16) return SX_ERR_INVALID;

  const CUtensorMapDataType dt = kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[3] = {(uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.za};
    uint64_t strides[2] = {(uint64_t)a.lda * elt, (uint64_t)a.a_plane_stride * elt};
    uint32_t box[3] = {(uint32_t)bk, 128u, 1u};
    int rc = encode_tensor_map_3d(&tmA, dt, a.A, dims, strides, box);
    if (rc != SX_OK) return rc;
  }
  if (a.b_mn) {
    uint64_t dims[3] = {(uint64_t)a.N, (uint64_t)a.K, (uint64_t)a.zb};
    uint64_t strides[2] = {(uint64_t)a.ldb * elt, (uint64_t)a.b_plane_stride * elt};
    uint32_t box[3] = {(uint32_t)(128 / elt), (uint32_t)bk, 1u};
    int rc = encode_tensor_map_3d(&tmB, dt, a.B, dims, strides, box);
    if (rc != SX_OK) return rc;
  } else {
    uint64_t dims[3] = {(uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.zb};
    uint64_t strides[2] = {(uint64_t)a.ldb * elt, (uint64_t)a.b_plane_stride * elt};
    uint32_t box[3] = {(uint32_t)bk, (uint32_t)bn, 1u};
    int rc = encode_tensor_map_3d(&tmB, dt, a.B, dims, strides, box);
    if (rc != SX_OK) return rc;
  }

  GemmParams p{};
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.batch = a.batch;
  p.nseg = a.nseg;
  for (int s = 0; s < 3; ++s) { p.a_plane[s] = a.a_plane[s]; p.b_plane[s] = a.b_plane[s]; }
  p.a_planes = a.a_planes; p.b_planes = a.b_planes;
  p.C = a.C; p.ldc = a.ldc; p.c_batch_stride = a.c_batch_stride;
  p.bias = a.bias; p.residual = a.residual;
  p.alpha = a.alpha; p.beta = a.beta; p.act = a.act;
  p.status = a.status;
  p.m_tiles = (int)((a.M + 127) / 128);
  p.n_tiles = (int)((a.N + bn - 1) / bn);
  p.group_m = a.group_m > 0 ? a.group_m : 8;
  p.wait_limit_ns = a.wait_limit_ns ? a.wait_limit_ns : WAIT_LIMIT_NS;
  p.fault_stop_early = a.fault_stop_early;

  const long long total = (long long)p.batch * p.m_tiles * p.n_tiles;
  const int grid = (int)(total < a.num_sms ? total : a.num_sms);

  if (kind == 0) {
    if (a.out_bf16) {
      return a.b_mn ? launch_bn<__nv_bfloat16, true, 0>(bn, tmA, tmB, p, grid, stream)
                    : launch_bn<__nv_bfloat16, false, 0>(bn, tmA, tmB, p, grid, stream);
    }
    return a.b_mn ? launch_bn<float, true, 0>(bn, tmA, tmB, p, grid, stream)
                  : launch_bn<float, false, 0>(bn, tmA, tmB, p, grid, stream);
  }
  return SX_ERR_INVALID;  // fp32 operands go through launch_gemm_tf32x3
}


KernelShape describe_gemm_tc(int bn) {
  auto mk = [](auto cfg) {
    using C = decltype(cfg);
    return KernelShape{"gemm_tc_kernel", C::BM, C::BN, C::BK, C::BM, C::BN, C::UMMA_K, 192, 1, C::STAGES, C::DYN_SMEM, C::TMEM_COLS};
  };
  return bn == 256 ? mk(TileCfg<256, 0>{}) : bn == 128 ? mk(TileCfg<128, 0>{}) : mk(TileCfg<64, 0>{});
}

}  // namespace sx
