// fp32 GEMM (3xTF32, round-to-nearest chunk accumulation) with the hi/lo operand split done INSIDE the kernel.
//
// gemm_tf32x3_kernel reads operands that a pre-pass has already split into {hi, lo} tf32 planes. That is the
// right trade for large products, where every plane is re-read by many tiles. For small and batched problems
// (512^3; 2048 x 64^3) each operand element is used by few tiles, the pre-pass triples the HBM traffic and adds
// two kernel launches. Here the TMA producer streams the RAW fp32 tiles; four converter warps turn each staged
// tile into the planes the tensor core consumes, in shared memory:
//   A tile  [128 rows][32 k], loaded 128B-swizzled: hi = tf32(x) overwrites x in place, lo = tf32(x - hi) goes
//           to a second buffer at the same (swizzled) position - the split is element-wise, so the swizzle
//           pattern carries over untouched.
//   B tile, column-major B ([N,K], K contiguous): same as A.
//   B tile, row-major B ([K,N]): loaded unswizzled as [32 k][64 n]; the converters transpose while splitting and
//           write K-major 128B-swizzled hi / lo tiles (kind::tf32 wants K-major operands here).
// Everything downstream (three MMAs per k step, main accumulator drained every 4 k-blocks into fp32 registers,
// correction accumulator added once per tile, fused epilogue) is the scheme of gemm_tf32x3_kernel.
//
//   warp 0      TMA producer (raw tiles)            warp 1      MMA issuer
//   warps 2..5  accumulate + epilogue               warps 6..13 converters
//
// Split-K over a thread-block cluster (kSplit = 2 or 4): when a problem has fewer tiles than a quarter (half)
// of the SMs but a long K, the per-k-block latency of this pipeline (TMA + conversion + MMA completion), not
// throughput, sets the run time. The kSplit CTAs of a cluster then work on the SAME output tile, each on its own
// contiguous range of k-blocks. Ranks 1.. park their fp32 partial tile in their own shared memory and signal the
// leader's mbarrier; the leader (rank 0) reads the partials over distributed shared memory (ld.shared::cluster),
// adds them in rank order - a fixed order, so results are reproducible - and runs the epilogue. All cross-CTA
// hand-offs are mbarriers with the same bounded waits as the pipeline; the only barrier.cluster is at kernel
// start (barrier initialisation visible cluster-wide) and at the end (nobody's shared memory goes away while a
// peer may still touch it), which every control path reaches.
#include <cuda_bf16.h>

#include <cstdlib>

#include "epilogue.cuh"
#include "gemm_params.h"
#include "host_api.h"
#include "options.h"
#include "sm100_ptx.cuh"

namespace sx {

template <int kSplit>
struct FusedCfgT {
  static constexpr int BM = 128, BN = 64, BK = 32, UMMA_K = 8, CHUNK_KB = 4;
  static constexpr int A_OFF = 0;             // raw A, becomes A hi          16 KB
  static constexpr int ALO_OFF = 16 * 1024;   // A lo                          16 KB
  static constexpr int BRAW_OFF = 32 * 1024;  // raw B (K-major: becomes hi)    8 KB
  static constexpr int BHI_OFF = 40 * 1024;   // B hi when B had to be transposed 8 KB
  static constexpr int BLO_OFF = 48 * 1024;   // B lo                           8 KB
  static constexpr int STAGE_BYTES = 56 * 1024;
  static constexpr int RAW_BYTES = 16 * 1024 + 8 * 1024;  // bytes the TMA delivers per stage
  static constexpr int STAGES = kSplit > 1 ? 3 : 4;         // split-K trades one stage for the partial-tile buffer
  static constexpr int PART_BYTES = kSplit > 1 ? BM * BN * 4 : 0;  // this CTA's fp32 partial tile (ranks 1..)
  static constexpr int TMEM_COLS = 4 * BN;  // main[2] + corr[2]
  static constexpr int CONV_WARPS = 8;                      // converter warps ...
  static constexpr int CONV_GROUPS = 2;                     // ... in groups that take alternate k-blocks
  static constexpr int THREADS = 192 + 32 * CONV_WARPS;
  static constexpr int DYN_SMEM = STAGES * STAGE_BYTES + PART_BYTES + 1024;
};
using FusedCfg = FusedCfgT<1>;

__device__ __forceinline__ float4 ld_shared_cluster_v4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr));  // volatile keeps it after the (volatile) barrier wait that precedes it
  return v;
}
__device__ __forceinline__ void mbar_arrive_cluster_relaxed_after(uint32_t cluster_addr, uint32_t dep) {
  asm volatile(
      "{\n"
      ".reg .pred q;\n"
      "setp.eq.u32 q, %1, 0xffffffff;\n"
      "@q mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];\n"
      "@!q mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];\n"
      "}\n" ::"r"(cluster_addr),
      "r"(dep)
      : "memory");
}

// Round to tf32 (10 mantissa bits), nearest with ties away from zero - the result of cvt.rna.tf32.f32, written
// with two full-rate integer instructions (add half an ulp to the magnitude, clear the 13 dropped bits) because
// the conversion instruction issues at a fraction of that rate and the converter warps are on the critical path.
__device__ __forceinline__ float tf32_rna(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}

__device__ __forceinline__ void split4(const float4& x, float4& hi, float4& lo) {
  hi.x = tf32_rna(x.x); hi.y = tf32_rna(x.y); hi.z = tf32_rna(x.z); hi.w = tf32_rna(x.w);
  lo.x = tf32_rna(x.x - hi.x); lo.y = tf32_rna(x.y - hi.y); lo.z = tf32_rna(x.z - hi.z); lo.w = tf32_rna(x.w - hi.w);
}

template <typename OutT, bool kBmn, int kSplit>
__global__ void __launch_bounds__(FusedCfg::THREADS, 1)
gemm_f32_fused_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const GemmParams p) {
  using Cfg = FusedCfgT<kSplit>;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES, CH = Cfg::CHUNK_KB;

  extern __shared__ uint8_t dyn_smem[];
  __shared__ uint64_t raw_full[STAGES], conv_done[STAGES], empty_bar[STAGES];
  __shared__ uint64_t main_full[2], main_empty[2], corr_full[2], corr_empty[2];
  // Split-K hand-off, one barrier per epilogue warp (32 rows of the tile): part_full[r - 1][q] lives in the
  // leader and is signalled by rank r; part_empty[q] lives in every rank >= 1 and is signalled by the leader.
  __shared__ uint64_t part_full[3][4], part_empty[4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&conv_done[s], Cfg::CONV_WARPS / Cfg::CONV_GROUPS);  // one arrival per converter warp of a group
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&main_full[a], 1);
      mbar_init(&main_empty[a], 4);
      mbar_init(&corr_full[a], 1);
      mbar_init(&corr_empty[a], 4);
    }
    for (int q = 0; q < 4; ++q) {
      mbar_init(&part_empty[q], 1);
      for (int r = 0; r < 3; ++r) mbar_init(&part_full[r][q], 1);
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
  if constexpr (kSplit > 1) cluster_sync_all();  // every CTA's barriers are initialised before a peer arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_launch_dependents();  // the next kernel in the stream may set itself up on SMs this grid leaves
  pdl_wait_prior_grids();   // the kernel before this one has completed: its outputs may be this one's operands

  const int per = p.m_tiles * p.n_tiles;
  const int total_tiles = p.batch * per;
  // This CTA's share of the k-blocks: the first (nkb_all mod kSplit) ranks take one more. The host only
  // splits when every rank gets at least one.
  const int rank = kSplit > 1 ? (int)cluster_ctarank() : 0;
  const int first_tile = blockIdx.x / kSplit, tile_step = gridDim.x / kSplit;
  const int nkb_all = (p.K + BK - 1) / BK;
  const int kb_base = nkb_all / kSplit, kb_rem = nkb_all % kSplit;
  const int kb0 = rank * kb_base + (rank < kb_rem ? rank : kb_rem);
  const int nkb = kb_base + (rank < kb_rem ? 1 : 0);
  const int nchunks = (nkb + CH - 1) / CH;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer: raw fp32 tiles
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = first_tile; ok && t < total_tiles; t += tile_step) {
        const int z = t / per, r = t - z * per;
        const int m0 = (r % p.m_tiles) * BM, n0 = (r / p.m_tiles) * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, &abort_flag)) { ok = false; break; }
          uint8_t* base = tiles + stage * Cfg::STAGE_BYTES;
          mbar_arrive_expect_tx(&raw_full[stage], Cfg::RAW_BYTES);
          const int k0 = (kb0 + kb) * BK;
          tma_load_3d(base + Cfg::A_OFF, &tmA, &raw_full[stage], k0, m0, z);
          if constexpr (kBmn) tma_load_3d(base + Cfg::BRAW_OFF, &tmB, &raw_full[stage], n0, k0, z);
          else tma_load_3d(base + Cfg::BRAW_OFF, &tmB, &raw_full[stage], k0, n0, z);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
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
      for (int t = first_tile; ok && t < total_tiles; t += tile_step) {
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
            const uint32_t base = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
            const uint32_t a_hi = base + Cfg::A_OFF, a_lo = base + Cfg::ALO_OFF;
            const uint32_t b_hi = base + (kBmn ? Cfg::BHI_OFF : Cfg::BRAW_OFF), b_lo = base + Cfg::BLO_OFF;
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
  } else if (warp >= 6) {
    // ------------------------------------------------------------ converters: two groups of four warps
    // A stage's conversion is a latency chain (wait, shared loads, split, shared stores, proxy fence, arrive), not
    // a throughput problem: eight warps on one stage were hardly faster than four. So the groups alternate
    // k-blocks - group g converts the k-blocks whose running index is congruent to g modulo 2 - and two stages
    // are in conversion at any time.
    constexpr int CT = 32 * Cfg::CONV_WARPS / Cfg::CONV_GROUPS;  // threads that share one stage
    const int group = (warp - 6) / (Cfg::CONV_WARPS / Cfg::CONV_GROUPS);
    const int tid = (threadIdx.x - 192) % CT;
    int it = 0;  // k-blocks this CTA has gone through, over all its tiles
    bool ok = true;
    for (int t = first_tile; ok && t < total_tiles; t += tile_step) {
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        if (it % Cfg::CONV_GROUPS != group) continue;
        const int stage = it % STAGES;
        const uint32_t phase = (uint32_t)(it / STAGES) & 1u;
        if (!mbar_wait(&raw_full[stage], phase, &abort_flag)) { ok = false; break; }
        uint8_t* base = tiles + stage * Cfg::STAGE_BYTES;
#pragma unroll
        for (int i = 0; i < 1024 / CT; ++i) {  // A: 1024 16-byte chunks, position-wise
          const int off = (i * CT + tid) * 16;
          float4 hi, lo;
          split4(*reinterpret_cast<const float4*>(base + Cfg::A_OFF + off), hi, lo);
          *reinterpret_cast<float4*>(base + Cfg::A_OFF + off) = hi;
          *reinterpret_cast<float4*>(base + Cfg::ALO_OFF + off) = lo;
        }
        if constexpr (!kBmn) {
#pragma unroll
          for (int i = 0; i < 512 / CT; ++i) {  // B [64 n][32 k], position-wise
            const int off = (i * CT + tid) * 16;
            float4 hi, lo;
            split4(*reinterpret_cast<const float4*>(base + Cfg::BRAW_OFF + off), hi, lo);
            *reinterpret_cast<float4*>(base + Cfg::BRAW_OFF + off) = hi;
            *reinterpret_cast<float4*>(base + Cfg::BLO_OFF + off) = lo;
          }
        } else {
          const float* raw = reinterpret_cast<const float*>(base + Cfg::BRAW_OFF);  // [32 k][64 n]
#pragma unroll
          for (int i = 0; i < 512 / CT; ++i) {  // transpose: 4 consecutive k of one column n -> one 16-byte chunk
            const int item = i * CT + tid;
            const int n = item & 63, kc = item >> 6;
            float4 x;
            x.x = raw[(kc * 4 + 0) * 64 + n];
            x.y = raw[(kc * 4 + 1) * 64 + n];
            x.z = raw[(kc * 4 + 2) * 64 + n];
            x.w = raw[(kc * 4 + 3) * 64 + n];
            float4 hi, lo;
            split4(x, hi, lo);
            const int off = n * 128 + ((kc ^ (n & 7)) << 4);
            *reinterpret_cast<float4*>(base + Cfg::BHI_OFF + off) = hi;
            *reinterpret_cast<float4*>(base + Cfg::BLO_OFF + off) = lo;
          }
        }
        fence_proxy_async_smem();  // the tensor core reads these tiles through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&conv_done[stage]);
      }
    }
  } else {
    // ------------------------------------------------------------ accumulate + epilogue (warps 2..5)
    const int q = warp & 3;
    const EpilogueCtx<OutT> ep(p);
    const uint32_t lane_base = uint32_t(q * 32) << 16;
    int macc = 0, cacc = 0;
    uint32_t mphase = 0, cphase = 0, xphase = 0;
    bool ok = true;
    for (int t = first_tile; ok && t < total_tiles; t += tile_step) {
      const int z = t / per, r = t - z * per;
      const int m0 = (r % p.m_tiles) * BM, n0 = (r / p.m_tiles) * BN;
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

      if constexpr (kSplit > 1) {
        // Partial tiles are laid out [16 column groups][128 rows][4 floats]: consecutive lanes (rows) touch
        // consecutive 16-byte chunks, for the writer and for the leader's remote reads alike.
        float* part = reinterpret_cast<float*>(tiles + STAGES * Cfg::STAGE_BYTES);
        const int prow = q * 32 + lane;
        if (rank != 0) {
          if (!mbar_wait<true>(&part_empty[q], xphase ^ 1, &abort_flag)) break;  // leader has read the previous one
#pragma unroll
          for (int g = 0; g < BN / 4; ++g)
            *reinterpret_cast<float4*>(part + (g * BM + prow) * 4) =
                make_float4(sum[g * 4 + 0], sum[g * 4 + 1], sum[g * 4 + 2], sum[g * 4 + 3]);
          __syncwarp();  // orders the other lanes' stores before lane 0's release
          if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&part_full[rank - 1][q]), 0));
          xphase ^= 1;
          continue;  // only the leader stores
        }
        bool got = true;
        for (int r = 1; r < kSplit; ++r)
          if (!mbar_wait<true>(&part_full[r - 1][q], xphase, &abort_flag)) { got = false; break; }
        if (got) {
          // Remote (distributed shared memory) loads take on the order of 100 ns each: a round issues the loads
          // of all peers for a group of columns before the first add, so 12 (8 for two CTAs) are in flight per
          // thread. The adds run in rank order per element, whatever the arrival order: reproducible bits.
          constexpr int G = kSplit == 2 ? 8 : 4;  // 16-byte column groups per peer and round
          uint32_t remote[kSplit - 1];
#pragma unroll
          for (int r = 1; r < kSplit; ++r) remote[r - 1] = mapa_u32(smem_u32(part), (uint32_t)r);
#pragma unroll
          for (int h = 0; h < BN / 4 / G; ++h) {
            float4 v[kSplit - 1][G];
#pragma unroll
            for (int r = 0; r < kSplit - 1; ++r)
#pragma unroll
              for (int g = 0; g < G; ++g)
                v[r][g] = ld_shared_cluster_v4(remote[r] + (uint32_t)(((h * G + g) * BM + prow) * 16));
#pragma unroll
            for (int r = 0; r < kSplit - 1; ++r)
#pragma unroll
              for (int g = 0; g < G; ++g) {
                const int j = (h * G + g) * 4;
                sum[j + 0] += v[r][g].x; sum[j + 1] += v[r][g].y; sum[j + 2] += v[r][g].z; sum[j + 3] += v[r][g].w;
              }
          }
          // Hand the buffers back only when the loads have returned: the sums they feed are folded into a vote
          // that the (relaxed: nothing to publish) remote arrives depend on - see mbar_arrive_after.
          uint32_t seen = 0;
#pragma unroll
          for (int j = 0; j < BN; ++j) seen |= __float_as_uint(sum[j]);
          const uint32_t vote = __ballot_sync(__activemask(), seen == 0x7fc0dead);
          if (lane == 0) {
#pragma unroll
            for (int r = 1; r < kSplit; ++r)
              mbar_arrive_cluster_relaxed_after(mapa_u32(smem_u32(&part_empty[q]), (uint32_t)r), vote);
          }
        }
        if (!got) break;
        xphase ^= 1;
      }

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
  if constexpr (kSplit > 1) cluster_sync_all();  // peers are done with this CTA's shared memory and barriers
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && abort_flag != 0 && p.status != nullptr) atomicExch(p.status, int(ST_WAIT_TIMEOUT));
}

// ------------------------------------------------------------------ host side
namespace {

template <typename OutT, bool kBmn, int kSplit>
int launch_fused(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid, cudaStream_t stream) {
  using Cfg = FusedCfgT<kSplit>;
  auto kern = gemm_f32_fused_kernel<OutT, kBmn, kSplit>;
  SX_ENSURE_DYN_SMEM(kern, Cfg::DYN_SMEM);
  return launch_kernel_ex(kern, (unsigned)grid, Cfg::THREADS, Cfg::DYN_SMEM, stream, kSplit, pdl_enabled(), tmA, tmB, p) ==
                 cudaSuccess
             ? SX_OK
             : SX_ERR_EXEC;
}

template <typename OutT, bool kBmn>
int launch_split(int split, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid,
                 cudaStream_t stream) {
  switch (split) {
    case 4: return launch_fused<OutT, kBmn, 4>(tmA, tmB, p, grid, stream);
    case 2: return launch_fused<OutT, kBmn, 2>(tmA, tmB, p, grid, stream);
    default: return launch_fused<OutT, kBmn, 1>(tmA, tmB, p, grid, stream);
  }
}

}  // namespace

bool f32_fused_operands_ok(const TcGemmArgs& a) {
  return a.lda % 4 == 0 && a.ldb % 4 == 0 && a.a_plane_stride % 4 == 0 && a.b_plane_stride % 4 == 0 &&
         reinterpret_cast<uintptr_t>(a.A) % 16 == 0 && reinterpret_cast<uintptr_t>(a.B) % 16 == 0;
}

// Raw fp32 operands: A [batch][M][lda]; B [batch][K][ldb] (a.b_mn = 1, row-major) or [batch][N][ldb] (a.b_mn = 0).
// a_plane_stride / b_plane_stride are the batch strides. Needs 16-byte aligned rows (f32_fused_operands_ok).
int launch_gemm_f32_fused(const TcGemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) return SX_ERR_INVALID;
  if (!f32_fused_operands_ok(a)) return SX_ERR_INVALID;
  if (f32_fused_tile_rows(a.M) == 64) return launch_gemm_f32_small(a, stream);  // at most 64 rows: its own kernel
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[3] = {(uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.batch};
    uint64_t strides[2] = {(uint64_t)a.lda * 4, (uint64_t)a.a_plane_stride * 4};
    uint32_t box[3] = {32u, 128u, 1u};
    int rc = encode_tensor_map_3d(&tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.A, dims, strides, box);
    if (rc != SX_OK) return rc;
  }
  if (a.b_mn) {
    uint64_t dims[3] = {(uint64_t)a.N, (uint64_t)a.K, (uint64_t)a.batch};
    uint64_t strides[2] = {(uint64_t)a.ldb * 4, (uint64_t)a.b_plane_stride * 4};
    uint32_t box[3] = {64u, 32u, 1u};
    int rc = encode_tensor_map_3d(&tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.B, dims, strides, box, /*swizzle128=*/false);
    if (rc != SX_OK) return rc;
  } else {
    uint64_t dims[3] = {(uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.batch};
    uint64_t strides[2] = {(uint64_t)a.ldb * 4, (uint64_t)a.b_plane_stride * 4};
    uint32_t box[3] = {32u, 64u, 1u};
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
  p.n_tiles = (int)((a.N + 63) / 64);
  const long long total = (long long)p.batch * p.m_tiles * p.n_tiles;
  const int split = f32_fused_split_k(total, a.K, a.num_sms);
  const long long clusters = total < a.num_sms / split ? total : a.num_sms / split;
  const int grid = (int)clusters * split;
  if (a.out_bf16)
    return a.b_mn ? launch_split<__nv_bfloat16, true>(split, tmA, tmB, p, grid, stream)
                  : launch_split<__nv_bfloat16, false>(split, tmA, tmB, p, grid, stream);
  return a.b_mn ? launch_split<float, true>(split, tmA, tmB, p, grid, stream)
                : launch_split<float, false>(split, tmA, tmB, p, grid, stream);
}

// Rows of one problem's output tile: 64 when the problem has at most 64 rows (gemm_f32_small_kernel takes it),
// else 128 (this file's kernel). The option "f32_tile_rows" = 128 forces this file's kernel (tests compare the two).
int f32_fused_tile_rows(long long M) {
  if (options().f32_tile_rows.load(std::memory_order_relaxed) == 128) return 128;
  return M <= 64 ? 64 : 128;
}


// How many CTAs share one output tile (split-K over a cluster): only when the tiles alone would leave most SMs
// idle and every rank still gets at least two k-blocks of 32.
int f32_fused_split_k(long long tiles, long long K, int num_sms) {
  {
    const int v = (int)options().f32_split_k.load(std::memory_order_relaxed);
    if (v == 1 || v == 2 || v == 4) return (K + 31) / 32 >= v ? v : 1;  // forced (tests): any tile count
  }
  const long long nkb = (K + 31) / 32;
  if (tiles * 4 <= num_sms && nkb >= 8) return 4;
  if (tiles * 2 <= num_sms && nkb >= 4) return 2;
  return 1;
}


KernelShape describe_gemm_f32_fused(int split) {
  auto mk = [](auto cfg, int cluster) {
    using C = decltype(cfg);
    return KernelShape{"gemm_f32_fused_kernel", C::BM, C::BN, C::BK, C::BM, C::BN, C::UMMA_K, C::THREADS, cluster, C::STAGES, C::DYN_SMEM, C::TMEM_COLS};
  };
  return split == 4 ? mk(FusedCfgT<4>{}, 4) : split == 2 ? mk(FusedCfgT<2>{}, 2) : mk(FusedCfgT<1>{}, 1);
}

}  // namespace sx
