// fp32 GEMM (3xTF32, round-to-nearest chunk accumulation) for batches of problems with at most 64 rows each
// (2048 x 64^3), where the run time should be HBM traffic and nothing else.
//
// Same arithmetic as gemm_f32_fused_kernel (raw fp32 tiles in, hi/lo split in shared memory, three MMAs per k
// step, main accumulator drained every 4 k-blocks), with two changes that only pay off for these shapes:
//   * TWO problems per tile. tcgen05.mma instructions that accumulate into the same tensor-memory tile run one
//     after the other, each with a latency of 50-100 ns however small it is; 24 of them per 64^3 product made
//     the fused kernel MMA-latency-bound (2.2 us per product, 44 % of the HBM roofline). Here a tile stacks the A
//     matrices of problems z and z+1 into 128 rows and puts their B matrices side by side as 128 columns: one
//     128 x 128 x 8 instruction then computes both products (the two diagonal 64 x 64 blocks of the accumulator;
//     the off-diagonal blocks are never read). Half the instructions per product; the wasted multiplies cost
//     nothing, the tensor pipe is idle most of the time anyway.
//   * decoupled rings. In the fused kernel a stage holds the raw tile AND its converted planes, so it is occupied
//     through load, conversion, MMA and MMA completion and only a fraction of the stages have a load in flight.
//     Here the TMA producer fills a ring of 2 RAW stages (32 KB: both problems' 64 x 32 of A and 32 x 64 of B)
//     that are released as soon as the converters have read them, and the converters write hi / lo planes into a
//     separate ring of 2 OPERAND stages (64 KB) that the MMA thread consumes.
//   * TMA-store epilogue. One thread owns one output row, so a direct 16-byte store instruction touches 32
//     different 128-byte lines; those stores and the converters' shared-memory traffic go through the same
//     load/store data pipe, which was the busiest unit of the fused kernel on these shapes. Final values are
//     staged as 32-row x 128-byte blocks in shared memory and leave through cp.async.bulk.tensor stores, which also
//     clip the ragged edges (M < 64, N not a multiple of 32). Falls back to direct stores when C is not 16-byte
//     aligned.
//
//   warp 0      TMA producer (raw ring)             warp 1      MMA issuer (operand ring)
//   warps 2..5  accumulate + epilogue               warps 6..13 converters, two groups on alternate k-blocks
#include <cuda_bf16.h>

#include <cstdlib>

#include "epilogue.cuh"
#include "gemm_params.h"
#include "host_api.h"
#include "options.h"
#include "sm100_ptx.cuh"

namespace sx {

struct SmallCfg {
  static constexpr int PM = 64, PN = 64;          // rows / columns of one problem's tile
  static constexpr int BM = 2 * PM, BN = 2 * PN;  // the MMA tile: two problems
  static constexpr int BK = 32, UMMA_K = 8, CHUNK_KB = 4;
  static constexpr int RAW_STAGES = 2, OP_STAGES = 2;
  static constexpr int RAW_A = 0, RAW_B = 16 * 1024, RAW_BYTES = 32 * 1024;
  static constexpr int OP_AHI = 0, OP_ALO = 16 * 1024, OP_BHI = 32 * 1024, OP_BLO = 48 * 1024, OP_BYTES = 64 * 1024;
  static constexpr int OP_BASE = RAW_STAGES * RAW_BYTES;
  static constexpr int TMEM_COLS = 4 * BN;  // main[2] + corr[2], 128 columns each
  static constexpr int CONV_WARPS = 8, CONV_GROUPS = 2;
  static constexpr int THREADS = 192 + 32 * CONV_WARPS;
  static constexpr int OUT_TILE = 32 * 128;                // one TMA-store block: 32 rows x 128 bytes, 128B-swizzled
  static constexpr int OUT_BASE = OP_BASE + OP_STAGES * OP_BYTES;
  static constexpr int OUT_BYTES = 4 * 2 * OUT_TILE;       // per epilogue warp: its 32 x 64 fp32 values = two blocks
  static constexpr int DYN_SMEM = RAW_STAGES * RAW_BYTES + OP_STAGES * OP_BYTES + OUT_BYTES + 1024;
  static_assert(DYN_SMEM <= 227 * 1024, "shared memory budget");
  static_assert(TMEM_COLS == 512, "tensor memory: all 512 columns");
};

// Round to tf32 (10 mantissa bits), nearest with ties away from zero - the result of cvt.rna.tf32.f32 - with two
// full-rate integer instructions.
__device__ __forceinline__ float small_tf32_rna(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}
__device__ __forceinline__ void small_split4(const float4& x, float4& hi, float4& lo) {
  hi.x = small_tf32_rna(x.x); hi.y = small_tf32_rna(x.y); hi.z = small_tf32_rna(x.z); hi.w = small_tf32_rna(x.w);
  lo.x = small_tf32_rna(x.x - hi.x); lo.y = small_tf32_rna(x.y - hi.y);
  lo.z = small_tf32_rna(x.z - hi.z); lo.w = small_tf32_rna(x.w - hi.w);
}


// Loads of a raw stage, volatile so that they stay where they are written (before the stage is handed back).
__device__ __forceinline__ float4 ld_raw_v4(const uint8_t* p) {
  float4 v;
  asm volatile("ld.volatile.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(smem_u32(p))
               : "memory");
  return v;
}
__device__ __forceinline__ float ld_raw_f32(const float* p) {
  float v;
  asm volatile("ld.volatile.shared.f32 %0, [%1];" : "=f"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}

template <typename OutT, bool kBmn>
__global__ void __launch_bounds__(SmallCfg::THREADS, 1)
gemm_f32_small_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using Cfg = SmallCfg;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, RS = Cfg::RAW_STAGES, OS = Cfg::OP_STAGES, CH = Cfg::CHUNK_KB;
  constexpr int PM = Cfg::PM, PN = Cfg::PN;

  extern __shared__ uint8_t dyn_smem[];
  __shared__ uint64_t raw_full[RS], raw_empty[RS], conv_done[OS], op_empty[OS];
  __shared__ uint64_t main_full[2], main_empty[2], corr_full[2], corr_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RS; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], Cfg::CONV_WARPS / Cfg::CONV_GROUPS);  // the converter warps of the group that read it
    }
    for (int s = 0; s < OS; ++s) {
      mbar_init(&conv_done[s], Cfg::CONV_WARPS / Cfg::CONV_GROUPS);
      mbar_init(&op_empty[s], 1);
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

  // A tile = one pair of problems (z0, z0 + 1) x one block of 64 columns. With an odd batch the last pair's
  // second half is loaded as zeros (TMA out-of-range fill) and never stored.
  const int per = p.n_tiles;
  const int total_tiles = ((p.batch + 1) / 2) * per;
  const int nkb = (p.K + BK - 1) / BK;
  const int nchunks = (nkb + CH - 1) / CH;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer: raw ring
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0, armed = 0, armed_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const int z0 = 2 * (t / per), n0 = (t % per) * PN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&raw_empty[stage], phase ^ 1, &abort_flag)) { ok = false; break; }
          uint8_t* base = tiles + stage * Cfg::RAW_BYTES;
          mbar_arrive_expect_tx(&raw_full[stage], Cfg::RAW_BYTES);
          armed |= 1u << stage;
          armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
          // boxes span two batch entries: [2][64][32] of A; [2][64 n][32 k] or [2][32 k][64 n] of B
          tma_load_3d(base + Cfg::RAW_A, &tmA, &raw_full[stage], kb * BK, 0, z0);
          if constexpr (kBmn) tma_load_3d(base + Cfg::RAW_B, &tmB, &raw_full[stage], n0, kb * BK, z0);
          else tma_load_3d(base + Cfg::RAW_B, &tmB, &raw_full[stage], kb * BK, n0, z0);
          if (++stage == RS) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok || abort_flag) {
        // Unwinding: give copies that were already issued a bounded time to land.
        const uint64_t t0 = globaltimer_ns();
        for (int s = 0; s < RS; ++s) {
          if (!(armed & (1u << s))) continue;
          while (!mbar_try_wait(&raw_full[s], (armed_phase >> s) & 1u)) {
            if (globaltimer_ns() - t0 > 2000000ull) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer: operand ring
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
            if (!mbar_wait(&conv_done[stage], phase, &abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t base = smem_u32(tiles + Cfg::OP_BASE + stage * Cfg::OP_BYTES);
            const uint32_t a_hi = base + Cfg::OP_AHI, a_lo = base + Cfg::OP_ALO;
            const uint32_t b_hi = base + Cfg::OP_BHI, b_lo = base + Cfg::OP_BLO;
#pragma unroll
            for (int k = 0; k < BK / Cfg::UMMA_K; ++k) {
              const uint32_t o = k * 32;
              umma<1, 1>(d_main, smem_desc(dhi, a_hi + o), smem_desc(dhi, b_hi + o), idesc, (kc | k) != 0 ? 1u : 0u);
              umma<1, 1>(d_corr, smem_desc(dhi, a_hi + o), smem_desc(dhi, b_lo + o), idesc, (kb | k) != 0 ? 1u : 0u);
              umma<1, 1>(d_corr, smem_desc(dhi, a_lo + o), smem_desc(dhi, b_hi + o), idesc, 1u);
            }
            umma_commit(&op_empty[stage]);
            if (++stage == OS) { stage = 0; phase ^= 1; }
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
  } else if (warp >= 6) {
    // ------------------------------------------------------------ converters: raw ring -> operand ring
    // Group g takes the k-blocks whose running index is congruent to g modulo 2, so two conversions (each a
    // latency chain of waits, shared loads, split, shared stores, proxy fence, arrive) overlap.
    constexpr int CT = 32 * Cfg::CONV_WARPS / Cfg::CONV_GROUPS;  // threads that share one k-block
    const int group = (warp - 6) / (Cfg::CONV_WARPS / Cfg::CONV_GROUPS);
    const int tid = (threadIdx.x - 192) % CT;
    int it = 0;  // k-blocks this CTA has gone through, over all its tiles
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        if (it % Cfg::CONV_GROUPS != group) continue;
        const int rs = it % RS, os = it % OS;
        if (!mbar_wait(&raw_full[rs], (uint32_t)(it / RS) & 1u, &abort_flag)) { ok = false; break; }
        if (!mbar_wait(&op_empty[os], ((uint32_t)(it / OS) & 1u) ^ 1u, &abort_flag)) { ok = false; break; }
        const uint8_t* raw = tiles + rs * Cfg::RAW_BYTES;
        uint8_t* op = tiles + Cfg::OP_BASE + os * Cfg::OP_BYTES;
        // Read the whole raw stage into registers first and hand it back to the producer at once: the next
        // load then overlaps the split arithmetic and the stores of this one.
        constexpr int NA = BM * 8 / CT, NB = BN * 8 / CT;
        float4 xa[NA], xb[NB];
#pragma unroll
        for (int i = 0; i < NA; ++i)  // A: 128 x 8 16-byte chunks, position-wise (the swizzle carries over)
          xa[i] = ld_raw_v4(raw + Cfg::RAW_A + (i * CT + tid) * 16);
        if constexpr (!kBmn) {
#pragma unroll
          for (int i = 0; i < NB; ++i)  // B [2 x 64 n][32 k], position-wise
            xb[i] = ld_raw_v4(raw + Cfg::RAW_B + (i * CT + tid) * 16);
        } else {
          const float* rb = reinterpret_cast<const float*>(raw + Cfg::RAW_B);  // [2][32 k][64 n], unswizzled
#pragma unroll
          for (int i = 0; i < NB; ++i) {  // transpose: 4 consecutive k of one column n -> one 16-byte chunk
            const int item = i * CT + tid;
            const int n = item & 63, kc = (item >> 6) & 7, b = item >> 9;
            const float* src = rb + b * (32 * 64) + kc * 4 * 64 + n;
            xb[i] = make_float4(ld_raw_f32(src), ld_raw_f32(src + 64), ld_raw_f32(src + 128), ld_raw_f32(src + 192));
          }
        }
        // The stage may be overwritten as soon as the producer sees the arrivals, but loads that are still in
        // flight are not waited for (see mbar_arrive_after): fold every load's result into one word, vote on it,
        // and make the arrive depend on the vote.
        uint32_t seen = 0;
#pragma unroll
        for (int i = 0; i < NA; ++i) seen |= __float_as_uint(xa[i].x) | __float_as_uint(xa[i].w);
#pragma unroll
        for (int i = 0; i < NB; ++i) seen |= __float_as_uint(xb[i].x) | __float_as_uint(xb[i].y) | __float_as_uint(xb[i].z) | __float_as_uint(xb[i].w);
        const uint32_t vote = __ballot_sync(__activemask(), seen == 0x7fc0dead);
        if (lane == 0) mbar_arrive_after(&raw_empty[rs], vote);  // the producer may refill the raw stage
#pragma unroll
        for (int i = 0; i < NA; ++i) {
          const int off = (i * CT + tid) * 16;
          float4 hi, lo;
          small_split4(xa[i], hi, lo);
          *reinterpret_cast<float4*>(op + Cfg::OP_AHI + off) = hi;
          *reinterpret_cast<float4*>(op + Cfg::OP_ALO + off) = lo;
        }
#pragma unroll
        for (int i = 0; i < NB; ++i) {
          int off = (i * CT + tid) * 16;
          if constexpr (kBmn) {
            const int item = i * CT + tid;
            const int n = item & 63, kc = (item >> 6) & 7, b = item >> 9;
            off = (b * 64 + n) * 128 + ((kc ^ (n & 7)) << 4);
          }
          float4 hi, lo;
          small_split4(xb[i], hi, lo);
          *reinterpret_cast<float4*>(op + Cfg::OP_BHI + off) = hi;
          *reinterpret_cast<float4*>(op + Cfg::OP_BLO + off) = lo;
        }
        fence_proxy_async_smem();  // the tensor core reads the planes through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&conv_done[os]);
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
    // Problem b = q / 2 of the pair: its rows are tensor-memory lanes 64 b .. 64 b + 63 (this warp: 32 of them) and
    // its product is the diagonal block, accumulator columns 64 b .. 64 b + 63.
    const int pb = q >> 1;
    const uint32_t col_base = uint32_t(pb * PN);
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      const int z = 2 * (t / per) + pb, n0 = (t % per) * PN;
      float sum[PN];
#pragma unroll
      for (int j = 0; j < PN; ++j) sum[j] = 0.0f;
      for (int ch = 0; ch < nchunks; ++ch) {
        if (!mbar_wait(&main_full[macc], mphase, &abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < PN / 32; ++c) {
          uint32_t rr[32];
          tmem_ld_32x32(tmem_base + lane_base + macc * BN + col_base + c * 32, rr);
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
      for (int c = 0; c < PN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32(tmem_base + lane_base + 2 * BN + cacc * BN + col_base + c * 32, rr);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[c * 32 + j] += __uint_as_float(rr[j]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&corr_empty[cacc]);
      if (++cacc == 2) { cacc = 0; cphase ^= 1; }

      const int row = (q & 1) * 32 + lane;
      const bool row_ok = z < p.batch && row < p.M;
      const long long row_off = (long long)z * p.c_batch_stride + (long long)row * p.ldc;
      if (p.n_dst != 0) {
        // Through shared memory and TMA stores: the warp's 32 x 64 values become one (bf16) or two (fp32) blocks of
        // 32 rows x 128 bytes, staged side by side, then one proxy fence and the stores. Rows >= M and columns >= N
        // are clipped by the tensor map. The blocks are reused a whole tile later, when their stores have long
        // been read out.
        constexpr int STRIPS = 128 / (32 * int(sizeof(OutT)));  // strips (32 columns) per 128-byte block: 1 or 2
        uint8_t* stg = tiles + Cfg::OUT_BASE + q * (2 * Cfg::OUT_TILE);
        if (lane == 0) bulk_wait_group_read<0>();
        __syncwarp();
        int nblk = 0;
#pragma unroll
        for (int c = 0; c < PN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = sum[c * 32 + j];
          ep.template math<false>(v, row_ok, row_off, col0);
          ep.stage(v, stg + (c / STRIPS) * Cfg::OUT_TILE, lane, (c % STRIPS) * (8 / STRIPS));
          nblk = c / STRIPS + 1;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && z < p.batch && (q & 1) * 32 < p.M) {  // skip blocks that lie entirely outside C
          for (int blk = 0; blk < nblk; ++blk)
            tma_store_3d(&tmC, stg + blk * Cfg::OUT_TILE, n0 + blk * STRIPS * 32, (q & 1) * 32, z);
          bulk_commit_group();
        }
      } else {
#pragma unroll
        for (int c = 0; c < PN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = sum[c * 32 + j];
          ep.template strip<false>(v, row_ok, row_off, col0);
        }
      }
    }
    if (p.n_dst != 0 && lane == 0) bulk_wait_group<0>();  // every store of this warp has been performed
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

template <typename OutT, bool kBmn>
int launch_small(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const GemmParams& p, int grid,
                 cudaStream_t stream) {
  auto kern = gemm_f32_small_kernel<OutT, kBmn>;
  SX_ENSURE_DYN_SMEM(kern, SmallCfg::DYN_SMEM);
  return launch_kernel_ex(kern, (unsigned)grid, SmallCfg::THREADS, SmallCfg::DYN_SMEM, stream, 1, pdl_enabled(), tmA, tmB,
                          tmC, p) == cudaSuccess
             ? SX_OK
             : SX_ERR_EXEC;
}

}  // namespace

// Raw fp32 operands with M <= 64 per problem (any batch; two problems share a tile): A [batch][M][lda]; B [batch][K][ldb] (a.b_mn = 1, row-major) or
// [batch][N][ldb] (a.b_mn = 0). Needs 16-byte aligned rows (f32_fused_operands_ok).
int launch_gemm_f32_small(const TcGemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.M > 64 || a.N <= 0 || a.K <= 0 || a.batch <= 0) return SX_ERR_INVALID;
  if (!f32_fused_operands_ok(a)) return SX_ERR_INVALID;
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[3] = {(uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.batch};
    uint64_t strides[2] = {(uint64_t)a.lda * 4, (uint64_t)a.a_plane_stride * 4};
    uint32_t box[3] = {32u, 64u, 2u};
    int rc = encode_tensor_map_3d(&tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.A, dims, strides, box);
    if (rc != SX_OK) return rc;
  }
  if (a.b_mn) {
    uint64_t dims[3] = {(uint64_t)a.N, (uint64_t)a.K, (uint64_t)a.batch};
    uint64_t strides[2] = {(uint64_t)a.ldb * 4, (uint64_t)a.b_plane_stride * 4};
    uint32_t box[3] = {64u, 32u, 2u};
    int rc = encode_tensor_map_3d(&tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.B, dims, strides, box, /*swizzle128=*/false);
    if (rc != SX_OK) return rc;
  } else {
    uint64_t dims[3] = {(uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.batch};
    uint64_t strides[2] = {(uint64_t)a.ldb * 4, (uint64_t)a.b_plane_stride * 4};
    uint32_t box[3] = {32u, 64u, 2u};
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
  p.m_tiles = 1;
  p.n_tiles = (int)((a.N + 63) / 64);
  // Output through TMA stores when C qualifies (16-byte aligned base, rows and batch stride); blocks of 32 rows x
  // 128 bytes. Otherwise the kernel stores directly and this map is a placeholder (a copy of A's).
  CUtensorMap tmC = tmA;
  const int elt = a.out_bf16 ? 2 : 4;
  if (reinterpret_cast<uintptr_t>(a.C) % 16 == 0 && (a.ldc * elt) % 16 == 0 && (a.c_batch_stride * elt) % 16 == 0 &&
      options().tma_store.load(std::memory_order_relaxed) != 0) {
    uint64_t dims[3] = {(uint64_t)a.N, (uint64_t)a.M, (uint64_t)a.batch};
    uint64_t strides[2] = {(uint64_t)a.ldc * elt, (uint64_t)a.c_batch_stride * elt};
    uint32_t box[3] = {(uint32_t)(128 / elt), 32u, 1u};
    int rc = encode_tensor_map_3d(&tmC, a.out_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.C,
                                  dims, strides, box);
    if (rc != SX_OK) return rc;
    p.n_dst = 1;
  }
  const long long total = (long long)((p.batch + 1) / 2) * p.n_tiles;
  const int grid = (int)(total < a.num_sms ? total : a.num_sms);
  if (a.out_bf16)
    return a.b_mn ? launch_small<__nv_bfloat16, true>(tmA, tmB, tmC, p, grid, stream)
                  : launch_small<__nv_bfloat16, false>(tmA, tmB, tmC, p, grid, stream);
  return a.b_mn ? launch_small<float, true>(tmA, tmB, tmC, p, grid, stream)
                : launch_small<float, false>(tmA, tmB, tmC, p, grid, stream);
}

KernelShape describe_gemm_f32_small() {
  using C = SmallCfg;
  // tile_m / tile_n: one problem's share of the 128 x 128 MMA tile
  return KernelShape{"gemm_f32_small_kernel", C::PM, C::PN, C::BK, C::BM, C::BN, C::UMMA_K, C::THREADS, 1,
                     C::RAW_STAGES, C::DYN_SMEM, C::TMEM_COLS};
}

}  // namespace sx
