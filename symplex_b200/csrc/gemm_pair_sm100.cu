// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2, one output tile per cluster of two CTAs.
//
// Why pairs: a CTA working alone on a 128x256 tile has to pull 48 KB of operands from L2 for every
// 4.2 MFLOP, which is more than the L2 -> SM path sustains at full tensor rate (measured: tensor pipe 66 %
// busy). In a pair each CTA stages only its own rows of A and HALF of the B tile; the paired MMA reads both
// halves. Two shapes, selected by kMB (128-row blocks of A per CTA):
//   kMB = 1   256 x 256 per pair, 32 KB / stage, 6 stages, TMEM = two alternating accumulators, so the
//             epilogue of tile t overlaps the main loop of tile t+1. Used when there are few tiles.
//   kMB = 2   512 x 256 per pair (256 x 256 per CTA), 48 KB / stage, 4 stages: 25 % less L2 -> SM traffic
//             per flop. TMEM holds the tile's two row blocks, so tiles cannot be double buffered; instead
//             the first and last two k-blocks of a tile are issued row-block-major, which lets the epilogue
//             of block 0 start 8 MMAs early and the next tile start on block 0 while block 1 is still
//             draining. Eight epilogue warps, all on block 0 first, then all on block 1.
//
// Roles per CTA: warp 0 = TMA producer for this CTA's tiles; warp 1 = TMEM allocation and, in the pair's
// leader (cluster rank 0) only, MMA issue for both CTAs; warps 2.. = epilogue for this CTA's rows.
// Barrier wiring: both producers' copies complete on the LEADER's full barrier; tcgen05.commit arrives on
// the empty / accumulator-full barriers of BOTH CTAs; epilogue warps release an accumulator with a
// (possibly remote) arrive on the leader's accumulator-empty barrier. No TMA multicast is used.
//
// Row-sharded products (kFwd instantiations): two more warps per CTA, the forwarders, copy every tile this CTA has
// finished from the local C (an L2 hit: the epilogue has just written it) to the same place in every other GPU's C,
// either with one 16-byte store per peer (XCHG_FORWARD) or with one multimem.st to a multicast mapping that the
// NVSwitch replicates (XCHG_MULTICAST). The local C is the buffer between the tensor pipe and NVLink, so link
// back-pressure delays only the forwarders, never the epilogue warps that must free tensor memory for the next tile.
// The ranks order themselves with flags written into each other's memory: READY (a rank has entered this call, its
// C may be overwritten) is awaited before the first remote store, DONE (all of a rank's tiles have landed) is
// written by the last forwarder warp of the grid and awaited by it, so the kernel ends only when the whole gathered
// C is in place on this GPU.
//
// Stream-K (kSK instantiations, 512 x 256 tiles): when the tiles do not fill the last wave of CTA pairs, the k-blocks
// of all tiles are laid out as one line and cut into one equal range per pair (PairWork below). A range that ends
// inside a tile leaves that tile's partial sums, raw fp32 straight from tensor memory, in the pair's slot of a
// workspace; the pair whose range holds the tile's last k-block adds them to its own accumulators in a fixed order
// (nearest pair first) and runs the epilogue. A pair writes its partial sums FIRST and adds other pairs' sums LAST, and
// only ever waits for pairs with a lower index, so the wait is over before it starts unless the grid is not
// co-resident, and even then it cannot deadlock while CTAs are dispatched in index order.
//
// All waits are bounded (sm100_ptx.cuh); on a timeout every role unwinds and the kernel reports
// ST_WAIT_TIMEOUT through the status word.
#include <cuda_bf16.h>

#include "epilogue.cuh"
#include "gemm_params.h"
#include "host_api.h"
#include "sm100_ptx.cuh"

namespace sx {

template <int kMB, bool kFwd = false>
struct PairCfg {
  static constexpr int ROWS = 128 * kMB;   // rows of A / C per CTA
  static constexpr int BM = 2 * ROWS;      // rows per pair
  static constexpr int BN = 256;
  static constexpr int BK = 64;            // 128 bytes of bf16
  static constexpr int UMMA_K = 16;
  static constexpr int A_BYTES = ROWS * 128;
  static constexpr int B_BYTES = 128 * 128;  // this CTA's 128 of the 256 columns
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = kMB == 1 ? 6 : 4;
  static constexpr int EPI_WARPS = 4 * kMB;
  // Forwarder warps copy finished tiles to the other GPUs (row-sharded products). The 256 x 256 shape, which the
  // link-bound calls take, has the registers for four of them (320 threads); the 512 x 256 shape for two (384).
  static constexpr int FWD_WARPS = kFwd ? (kMB == 1 ? 4 : 2) : 0;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS + 32 * FWD_WARPS;
  static constexpr int TMEM_COLS = 512;  // two 256-column accumulators
  static constexpr int STAGING_BYTES = 32 * 128;  // per epilogue warp: 32 rows x 128 bytes, 128B-swizzled
  static constexpr int DYN_SMEM = STAGES * STAGE_BYTES + EPI_WARPS * STAGING_BYTES + 1024;
};

struct DstMaps {
  CUtensorMap m[MAX_DST];
};

struct PairTile {
  int z, m0, n0;
};

template <int BM, int BN>
__device__ __forceinline__ PairTile pair_tile(const GemmParams& p, int t) {
  const int per = p.m_tiles * p.n_tiles;
  const int z = t / per;
  const int r = t - z * per;
  const int band = p.group_m * p.n_tiles;
  const int g = r / band;
  const int first_m = g * p.group_m;
  const int gsz = min(p.m_tiles - first_m, p.group_m);
  const int in_band = r - g * band;
  PairTile c;
  c.z = z;
  c.m0 = (first_m + in_band % gsz) * BM;
  c.n0 = (in_band / gsz) * BN;
  return c;
}

// The work of one CTA pair, item by item: (tile, k-blocks [kb0, kb1), kind).
enum WorkKind : int { WORK_FULL = 0, WORK_PARTIAL = 1, WORK_OWNER = 2 };
constexpr int SK_GRAIN = 4;  // range boundaries are multiples of this many k-blocks

// First unit (tile * nkb + k-block) of pair q's range; q == pairs gives the end of the line.
__host__ __device__ __forceinline__ long long sk_start(long long total_units, int pairs, int q) {
  if (q >= pairs) return total_units;
  return (total_units * q / pairs) / SK_GRAIN * SK_GRAIN;
}

template <bool kSK>
struct PairWork {
  int t, kb0, kb1, kind;  // the current item; t < 0: no more work
  // whole tiles, strided (no stream-K) or consecutive (stream-K)
  int next_full, end_full, stride, nkb;
  // stream-K: the range's partial first tile (owner) and partial last tile (contributor)
  int own_t, own_k0, part_t, part_k0, part_k1, stage;

  __host__ __device__ PairWork(int pair_id, int num_pairs, int total_tiles, int nkb_) : nkb(nkb_) {
    kb0 = 0;
    kb1 = nkb;
    kind = WORK_FULL;
    own_t = part_t = -1;
    own_k0 = part_k0 = part_k1 = 0;
    stage = 0;
    if constexpr (!kSK) {
      next_full = pair_id;
      end_full = total_tiles;
      stride = num_pairs;
    } else {
      stride = 1;
      const long long total = (long long)total_tiles * nkb;
      const long long u0 = sk_start(total, num_pairs, pair_id), u1 = sk_start(total, num_pairs, pair_id + 1);
      const int ta = int(u0 / nkb), ka = int(u0 - (long long)ta * nkb);
      const int tb = int(u1 / nkb), kbe = int(u1 - (long long)tb * nkb);
      if (ta == tb) {  // inside one tile and short of its end
        next_full = end_full = 0;
        if (u1 > u0) { part_t = ta; part_k0 = ka; part_k1 = kbe; }
      } else {
        if (kbe > 0) { part_t = tb; part_k0 = 0; part_k1 = kbe; }
        if (ka > 0) { own_t = ta; own_k0 = ka; }
        next_full = ka > 0 ? ta + 1 : ta;
        end_full = tb;
      }
    }
    next();
  }
  __host__ __device__ bool valid() const { return t >= 0; }
  __host__ __device__ void next() {
    if constexpr (!kSK) {
      t = next_full < end_full ? next_full : -1;
      next_full += stride;
    } else {
      // order: the contribution to another pair's tile, whole tiles, the tile that needs other pairs' contributions
      if (stage == 0) {
        stage = 1;
        if (part_t >= 0) { t = part_t; kb0 = part_k0; kb1 = part_k1; kind = WORK_PARTIAL; return; }
      }
      if (stage == 1) {
        if (next_full < end_full) { t = next_full++; kb0 = 0; kb1 = nkb; kind = WORK_FULL; return; }
        stage = 2;
      }
      if (stage == 2) {
        stage = 3;
        if (own_t >= 0) { t = own_t; kb0 = own_k0; kb1 = nkb; kind = WORK_OWNER; return; }
      }
      t = -1;
    }
  }
};

template <typename OutT, bool kBmn, int kMB, bool kFwd, bool kSK>
__global__ void __launch_bounds__(PairCfg<kMB, kFwd>::THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ DstMaps dst, const GemmParams p) {
  using Cfg = PairCfg<kMB, kFwd>;
  constexpr int BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES;

  extern __shared__ uint8_t dyn_smem[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint64_t fwd_bar[Cfg::EPI_WARPS];  // per epilogue warp: a finished block is back in its staging tile
  __shared__ uint32_t tmem_base_slot;
  __shared__ uint32_t stored_warps;  // kFwd: epilogue warps x tiles whose stores to the local C have been performed
  __shared__ int abort_flag;

  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();  // 0 = leader
  const uint64_t wait_ns = p.wait_limit_ns;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);   // leader: its producer's arrive.expect_tx (bytes of both CTAs)
      mbar_init(&empty_bar[s], 1);  // one tcgen05.commit per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8 * kMB);  // every epilogue warp of both CTAs releases each accumulator
    }
    for (int w = 0; w < Cfg::EPI_WARPS; ++w) mbar_init(&fwd_bar[w], 1);
    abort_flag = 0;
    stored_warps = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<2>(&tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish<2>();
  }
  tc_fence_before_sync();
  __syncwarp();  // the cluster barrier is warp-aligned: reconverge after the single-thread setup above
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_launch_dependents();  // the next kernel in the stream may set itself up on SMs this grid leaves
  pdl_wait_prior_grids();   // the kernel before this one has completed: its outputs may be this one's operands

  const int total_tiles = p.batch * p.m_tiles * p.n_tiles;
  const int nkb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0, armed_phase = 0;  // leader: stages whose copies (of both CTAs) may still be in flight
      bool ok = true;
      for (PairWork<kSK> w(pair_id, num_pairs, total_tiles, nkb); ok && w.valid(); w.next()) {
        const PairTile tc = pair_tile<Cfg::BM, BN>(p, w.t);
        const int my_m0 = tc.m0 + int(cta_rank) * Cfg::ROWS;
        const int my_n0 = tc.n0 + int(cta_rank) * 128;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, &abort_flag, wait_ns)) { ok = false; break; }
          uint8_t* sa = tiles + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          if (cta_rank == 0) {
            mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::STAGE_BYTES);
            armed |= 1u << stage;
            armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
          }
          const uint32_t leader_full = mapa_u32(smem_u32(&full_bar[stage]), 0);
          tma_load_3d_pair(sa, &tmA, leader_full, kb * BK, my_m0, tc.z);  // ROWS x 64 box
          if constexpr (kBmn) {
            tma_load_3d_pair(sb, &tmB, leader_full, my_n0, kb * BK, tc.z);
            tma_load_3d_pair(sb + BK * 128, &tmB, leader_full, my_n0 + 64, kb * BK, tc.z);
          } else {
            tma_load_3d_pair(sb, &tmB, leader_full, kb * BK, my_n0, tc.z);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Unwinding: copies that were already issued get a bounded time to land before the CTAs leave. The leader
        // sees both CTAs' bytes on its full barriers; its partner, which has no barrier of its own to watch, gives
        // its copies a fixed grace period (a copy takes a few microseconds) and then meets the leader at the
        // cluster barrier below.
        const uint64_t t0 = globaltimer_ns();
        if (cta_rank == 0) {
          for (int s = 0; s < STAGES; ++s) {
            if (!(armed & (1u << s))) continue;
            while (!mbar_try_wait(&full_bar[s], (armed_phase >> s) & 1u)) {
              if (globaltimer_ns() - t0 > 2000000ull) break;
            }
          }
        } else {
          while (globaltimer_ns() - t0 < 100000ull) __nanosleep(1000);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc(1, false, kBmn, 256, BN);
      constexpr uint64_t a_hi = make_smem_desc_hi(16, 1024);
      // B half tile held MN-major: two boxes of [64 k][64 n] (8192 B apart), 8-row k groups 1024 B apart.
      constexpr uint64_t b_hi = kBmn ? make_smem_desc_hi(BK * 128, 1024) : make_smem_desc_hi(16, 1024);
      constexpr uint32_t b_kstep = kBmn ? Cfg::UMMA_K * 128 : 32;
      constexpr int KSTEPS = BK / Cfg::UMMA_K;
      int stage = 0;
      uint32_t phase = 0;
      int slot = 0;            // kMB == 1: accumulator used by this tile
      uint32_t acc_phase = 0;  // kMB == 1: flips every second tile; kMB == 2: every tile
      bool ok = true;
      auto advance = [&](int& s, uint32_t& ph) {
        if (++s == STAGES) { s = 0; ph ^= 1; }
      };
      // four MMAs (one 64-wide k-block) into accumulator `mb` from stage `s`
      auto issue_block = [&](int mb, int s, uint32_t accumulate) {
        const uint32_t a_addr = smem_u32(tiles + s * Cfg::STAGE_BYTES) + mb * (128 * 128);
        const uint32_t b_addr = smem_u32(tiles + s * Cfg::STAGE_BYTES) + Cfg::A_BYTES;
#pragma unroll
        for (int k = 0; k < KSTEPS; ++k)
          umma<2, 0>(tmem_base + mb * BN, smem_desc(a_hi, a_addr + k * 32), smem_desc(b_hi, b_addr + k * b_kstep),
                     idesc, accumulate | (k != 0 ? 1u : 0u));
      };
      for (PairWork<kSK> w(pair_id, num_pairs, total_tiles, nkb); ok && w.valid(); w.next()) {
        const int nk = w.kb1 - w.kb0;  // k-blocks of this item, counted from 0 below
        if constexpr (kMB == 1) {
          if (!mbar_wait<true>(&acc_empty[slot], acc_phase ^ 1, &abort_flag, wait_ns)) break;
          tc_fence_after_sync();
          for (int kb = 0; kb < nk; ++kb) {
            if (!mbar_wait(&full_bar[stage], phase, &abort_flag, wait_ns)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t a_addr = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
            const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k)
              umma<2, 0>(tmem_base + slot * BN, smem_desc(a_hi, a_addr + k * 32),
                         smem_desc(b_hi, b_addr + k * b_kstep), idesc, (kb | k) != 0 ? 1u : 0u);
            umma_commit_pair(&empty_bar[stage], 3);  // frees this stage in both CTAs
            advance(stage, phase);
          }
          if (!ok) break;
          umma_commit_pair(&acc_full[slot], 3);
          if (++slot == 2) { slot = 0; acc_phase ^= 1; }
        } else {
          // The tile's two row blocks share every B stage. In the middle of a tile their MMAs interleave; the
          // first and the last SKEW k-blocks are issued block-major, so block 0 completes 4*SKEW MMAs before
          // block 1 and the next tile can start on block 0 while block 1 is still being drained.
          constexpr int SKEW = 2;
          const int head_end = min(SKEW, nk);
          const int tail_begin = max(head_end, nk - SKEW);
          auto group = [&](int g0, int g1) {  // k-blocks [g0, g1) block-major
            for (int mb = 0; mb < 2 && ok; ++mb) {
              if (g0 == 0) {
                if (!mbar_wait<true>(&acc_empty[mb], acc_phase ^ 1, &abort_flag, wait_ns)) { ok = false; break; }
                tc_fence_after_sync();
              }
              int s = stage;
              uint32_t ph = phase;
              for (int kb = g0; kb < g1; ++kb) {
                if (mb == 0) {
                  if (!mbar_wait(&full_bar[s], ph, &abort_flag, wait_ns)) { ok = false; break; }
                  tc_fence_after_sync();
                }
                issue_block(mb, s, kb != 0 ? 1u : 0u);
                if (mb == 1) umma_commit_pair(&empty_bar[s], 3);
                advance(s, ph);
              }
              if (ok && g1 == nk) umma_commit_pair(&acc_full[mb], 3);
            }
            for (int kb = g0; kb < g1; ++kb) advance(stage, phase);
          };
          group(0, head_end);
          for (int kb = head_end; ok && kb < tail_begin; ++kb) {
            if (!mbar_wait(&full_bar[stage], phase, &abort_flag, wait_ns)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t a_addr = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
            const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k) {
#pragma unroll
              for (int mb = 0; mb < 2; ++mb)
                umma<2, 0>(tmem_base + mb * BN, smem_desc(a_hi, a_addr + mb * (128 * 128) + k * 32),
                           smem_desc(b_hi, b_addr + k * b_kstep), idesc, 1u);
            }
            umma_commit_pair(&empty_bar[stage], 3);
            advance(stage, phase);
          }
          if (ok && tail_begin < nk) group(tail_begin, nk);
          if (!ok) break;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp < 2 + Cfg::EPI_WARPS) {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    // kMB == 1: four warps, each drains all 256 columns of the tile's accumulator.
    // kMB == 2: eight warps drain block 0 and then block 1, each taking one half of the columns, so block 0 is
    //           free again after half the epilogue time.
    const int half = kMB == 1 ? 0 : (warp - 2) >> 2;
    constexpr int STRIPS = (BN / 32) / kMB;  // 32-column strips per warp and accumulator
    const EpilogueCtx<OutT> ep(p);
    uint8_t* staging = tiles + STAGES * Cfg::STAGE_BYTES + (warp - 2) * Cfg::STAGING_BYTES;
    int slot = 0;
    uint32_t acc_phase = 0, fwd_phase = 0;
    bool ok = true;
    // Stream-K: this warp's chunks (32 rows x 32 columns of fp32, lane-interleaved float4s) inside a pair's slot of the
    // workspace, and its flag word. A warp only ever exchanges partial sums with the same warp of the same CTA rank
    // of another pair, which drains the same part of the tile.
    constexpr int SK_CHUNK = 32 * 32;  // floats
    constexpr int SK_SLOT = 2 * kMB * Cfg::EPI_WARPS * STRIPS * SK_CHUNK;
    const int sk_warp_word = int(cta_rank) * Cfg::EPI_WARPS + (warp - 2);
    auto sk_chunk = [&](int pair, int blk, int c) -> float* {
      return p.sk_ws + (long long)pair * SK_SLOT +
             (((int(cta_rank) * kMB + blk) * Cfg::EPI_WARPS + (warp - 2)) * STRIPS + (c - half * STRIPS)) * SK_CHUNK + lane * 4;
    };
    auto sk_dump = [&](const uint32_t (&r)[32], float* dst) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        st_global_v4(dst + j * 128, make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]));
    };
    auto sk_add = [&](float (&v)[32], int contributors, int blk, int c) {
      for (int i = 0; i < contributors; ++i) {  // fixed order: the nearest pair first
        const float* src = sk_chunk(pair_id - 1 - i, blk, c);
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // four 16-byte loads in flight per lane
          uint4 x[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) x[j] = ld_global_cg_v4(src + (4 * h + j) * 128);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[16 * h + 4 * j] += __uint_as_float(x[j].x);
            v[16 * h + 4 * j + 1] += __uint_as_float(x[j].y);
            v[16 * h + 4 * j + 2] += __uint_as_float(x[j].z);
            v[16 * h + 4 * j + 3] += __uint_as_float(x[j].w);
          }
        }
      }
    };
    for (PairWork<kSK> w(pair_id, num_pairs, total_tiles, nkb); ok && w.valid(); w.next()) {
      const PairTile tc = pair_tile<Cfg::BM, BN>(p, w.t);
      int contributors = 0;  // stream-K, WORK_OWNER: pairs whose partial sums belong to this tile
      if constexpr (kSK) {
        if (w.kind == WORK_OWNER) {
          const long long total = (long long)total_tiles * nkb, tile_u0 = (long long)w.t * nkb;
          for (int q = pair_id - 1; q >= 0 && sk_start(total, num_pairs, q + 1) > tile_u0; --q) ++contributors;
          for (int i = lane; i < contributors; i += 32)
            ok = ok && flag_wait_ge_gpu(p.sk_flags + (pair_id - 1 - i) * (2 * Cfg::EPI_WARPS) + sk_warp_word, p.sk_epoch,
                                        &abort_flag, wait_ns);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
      }
#pragma unroll 1
      for (int blk = 0; blk < kMB; ++blk) {
        if constexpr (kMB == 2) slot = blk;
        if (!mbar_wait(&acc_full[slot], acc_phase, &abort_flag, wait_ns)) { ok = false; break; }
        tc_fence_after_sync();
        const int row0 = tc.m0 + int(cta_rank) * Cfg::ROWS + blk * 128 + q * 32;  // this warp's first row
        const int row = row0 + lane;
        const bool row_ok = row < p.M;
        const long long row_off = (long long)tc.z * p.c_batch_stride + (long long)row * p.ldc;
#pragma unroll 1
        for (int c = half * STRIPS; c < (half + 1) * STRIPS; c += 2) {
          // two 32-column strips per wait: the second load's latency hides behind the first strip's math
          uint32_t r0[32], r1[32];
          const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + slot * BN + c * 32;
          tmem_ld_32x32(taddr, r0);
          tmem_ld_32x32(taddr + 32, r1);
          tmem_ld_wait();
          if constexpr (kSK) {
            if (w.kind == WORK_PARTIAL) {  // raw partial sums, whatever part of them lies inside C
              sk_dump(r0, sk_chunk(pair_id, blk, c));
              sk_dump(r1, sk_chunk(pair_id, blk, c + 1));
              continue;
            }
          }
          const int col0 = tc.n0 + c * 32;
          if (col0 >= p.N) continue;
          const bool second = col0 + 32 < p.N;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r0[j]);
          if constexpr (kSK) sk_add(v, contributors, blk, c);
          ep.template math<true>(v, row_ok, row_off, col0);
          if (p.n_dst == 0) {
            ep.store(v, row_ok, row_off, col0);
            if (!second) continue;
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r1[j]);
            if constexpr (kSK) sk_add(v, contributors, blk, c + 1);
            ep.template strip<true>(v, row_ok, row_off, col0 + 32);
          } else {
            // Staged path: the warp's 32 x 128-byte block goes to shared memory and one lane hands it to the
            // TMA unit, which writes it to the local C. bf16: both strips form one block; fp32: one block
            // per strip. (Peers are served after TMEM has been released, see below.)
            if (lane == 0) bulk_wait_group_read<0>();  // the previous block has left the staging tile
            __syncwarp();
            ep.stage(v, staging, lane, 0);
            if constexpr (sizeof(OutT) == 4) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&dst.m[0], staging, col0, row0, tc.z);
                bulk_commit_group();
              }
              if (!second) continue;
            }
            if (second) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r1[j]);
              if constexpr (kSK) sk_add(v, contributors, blk, c + 1);
              ep.template math<true>(v, row_ok, row_off, col0 + 32);
              if constexpr (sizeof(OutT) == 4) {
                if (lane == 0) bulk_wait_group_read<0>();
                __syncwarp();
                ep.stage(v, staging, lane, 0);
              } else {
                ep.stage(v, staging, lane, 4);
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const int cstore = sizeof(OutT) == 4 ? col0 + 32 : col0;
              tma_store_3d(&dst.m[0], staging, cstore, row0, tc.z);
              bulk_commit_group();
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[slot]), 0));  // leader's barrier
      }
      if constexpr (kMB == 1) {
        if (++slot == 2) { slot = 0; acc_phase ^= 1; }
      } else {
        acc_phase ^= 1;
      }
      if constexpr (kSK) {
        if (ok && w.kind == WORK_PARTIAL) {  // this warp's part of the partial sums is in the workspace
          __threadfence();
          __syncwarp();
          if (lane == 0) flag_store_release_gpu(p.sk_flags + pair_id * (2 * Cfg::EPI_WARPS) + sk_warp_word, p.sk_epoch);
        }
      }
      if constexpr (kFwd) {
        // Tell the forwarder warps that this warp's part of the tile is in the local C.
        if (lane == 0) {
          bulk_wait_group<0>();  // the stores have been performed
          smem_counter_add_release(&stored_warps, 1u);
        }
      }
      // XCHG_EPILOGUE_TMA: forwarding to the peer GPUs by this warp. TMEM is free again, so the MMAs of the next
      // tile are already running. Each block this warp wrote to the local C is read back (an L2 hit) into the
      // staging tile by TMA and stored to every peer's C.
      if (ok && p.n_dst > 1) {
        if (lane == 0) {
          bulk_wait_group<0>();  // this tile's local stores have been performed
          constexpr int STEP = sizeof(OutT) == 4 ? 1 : 2;  // strips per 128-byte block
          for (int blk = 0; ok && blk < kMB; ++blk) {
            const int row0 = tc.m0 + int(cta_rank) * Cfg::ROWS + blk * 128 + q * 32;
            if (row0 >= p.M) continue;
            for (int c = half * STRIPS; c < (half + 1) * STRIPS; c += STEP) {
              const int col0 = tc.n0 + c * 32;
              if (col0 >= p.N) break;
              bulk_wait_group_read<0>();  // the previous block has left the staging tile
              mbar_arrive_expect_tx(&fwd_bar[warp - 2], Cfg::STAGING_BYTES);
              tma_load_3d(staging, &dst.m[0], &fwd_bar[warp - 2], col0, row0, tc.z);
              if (!mbar_wait(&fwd_bar[warp - 2], fwd_phase, &abort_flag, wait_ns)) { ok = false; break; }
              fwd_phase ^= 1;
              for (int d = 1; d < p.n_dst; ++d) tma_store_3d(&dst.m[d], staging, col0, row0, tc.z);
              bulk_commit_group();
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
    }
    if (p.n_dst != 0 && lane == 0) bulk_wait_group<0>();  // every store of this warp has been performed
  } else if constexpr (kFwd) {
    // ------------------------------------------------------------ forwarders (both CTAs)
    const int fw = warp - 2 - Cfg::EPI_WARPS;
    const int np = p.n_peers;
    bool ok = true;
    // Entering the call: this GPU's earlier work on the stream is complete, so the peers may overwrite its C.
    if (blockIdx.x == 0 && fw == 0 && lane < np) flag_store_release_sys(p.peer_flags[lane] + FLAG_READY + p.my_rank, p.epoch);
    // No remote store before every peer has entered the call.
    if (lane < np) ok = flag_wait_ge(p.flags + FLAG_READY + p.peer_rank[lane], p.epoch, &abort_flag, wait_ns);
    ok = __all_sync(0xffffffffu, ok);
    constexpr int ROW_BYTES = BN * int(sizeof(OutT));  // this CTA's rows of a tile are ROW_BYTES wide
    constexpr int CH = ROW_BYTES / 512;                // 16-byte chunks per lane and row
    constexpr int U = 8 / CH;                          // rows per round: 8 loads in flight per lane
    uint8_t* const cbase = reinterpret_cast<uint8_t*>(p.C);
    uint32_t done_tiles = 0;
    for (int t = pair_id; ok && t < total_tiles; t += num_pairs) {
      ++done_tiles;
      if (lane == 0) ok = smem_counter_wait_ge(&stored_warps, done_tiles * Cfg::EPI_WARPS, &abort_flag, wait_ns);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      __syncwarp();
      if (!ok) break;
      const PairTile tc = pair_tile<Cfg::BM, BN>(p, t);
      const int row_base = tc.m0 + int(cta_rank) * Cfg::ROWS;
      const long long tile_off = ((long long)tc.z * p.c_batch_stride + tc.n0) * (long long)sizeof(OutT);
      // Rounds of U rows, software-pipelined: the loads of the next round are in flight while this round is stored.
      auto load_round = [&](int r, uint4 (&v)[U][CH], long long (&off)[U][CH]) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int ch = 0; ch < CH; ++ch) {
            const int row = row_base + r + u;
            const int colb = ch * 512 + lane * 16;
            const bool in = row < p.M && tc.n0 + colb / int(sizeof(OutT)) < p.N;  // rows are 16-byte multiples
            off[u][ch] = in ? tile_off + (long long)row * p.ldc * (long long)sizeof(OutT) + colb : -1;  // -1: outside C
            if (in) v[u][ch] = ld_global_cg_v4(cbase + off[u][ch]);
          }
        }
      };
      auto store_round = [&](const uint4 (&v)[U][CH], const long long (&off)[U][CH]) {
        if (p.xchg == XCHG_MULTICAST) {
          uint8_t* const mc = reinterpret_cast<uint8_t*>(p.mc_C);
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int ch = 0; ch < CH; ++ch)
              if (off[u][ch] >= 0) multimem_st_v4(mc + off[u][ch], v[u][ch]);
        } else {
          for (int d = 0; d < np; ++d) {
            uint8_t* const pc = reinterpret_cast<uint8_t*>(p.peer_C[d]);
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
              for (int ch = 0; ch < CH; ++ch)
                if (off[u][ch] >= 0) st_global_v4(pc + off[u][ch], v[u][ch]);
          }
        }
      };
      constexpr int STEP = Cfg::FWD_WARPS * U;
      uint4 va[U][CH], vb[U][CH];
      long long oa[U][CH], ob[U][CH];
      int r = fw * U;
      bool have = r < Cfg::ROWS && row_base + r < p.M;
      if (have) load_round(r, va, oa);
      while (have) {
        const int rn = r + STEP;
        const bool next = rn < Cfg::ROWS && row_base + rn < p.M;
        if (next) load_round(rn, vb, ob);
        store_round(va, oa);
        if (next) {
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
              va[u][ch] = vb[u][ch];
              oa[u][ch] = ob[u][ch];
            }
        }
        r = rn;
        have = next;
      }
    }
    // Completion. Every forwarder warp checks in (also after a failure, so the counter returns to zero); the last
    // one of the grid knows that all of this GPU's tiles are on their way, orders them before the DONE flags it
    // writes to the peers, and waits for the peers' DONE flags: when the kernel ends, the gathered C is complete.
    __threadfence_system();
    __syncwarp();
    // Low half of the counter: warps that have checked in; high half: how many of them gave up.
    const bool failed = !ok || *reinterpret_cast<volatile int*>(&abort_flag) != 0;
    uint32_t prev = 0;
    if (lane == 0) prev = atomicAdd(p.xchg_counter, 1u + (failed ? 0x10000u : 0u));
    prev = __shfl_sync(0xffffffffu, prev, 0);
    if ((prev & 0xffffu) == gridDim.x * Cfg::FWD_WARPS - 1) {
      if (lane == 0) *p.xchg_counter = 0;
      __threadfence_system();
      // A failure anywhere on this GPU withholds DONE: the peers' waits then run out as well, and every rank's
      // status word reports it.
      const bool good = !failed && (prev >> 16) == 0;
      if (good && lane < np) flag_store_release_sys(p.peer_flags[lane] + FLAG_DONE + p.my_rank, p.epoch);
      if (good && lane < np) flag_wait_ge(p.flags + FLAG_DONE + p.peer_rank[lane], p.epoch, &abort_flag, wait_ns);
    }
  }

  // Both CTAs stay resident until every remote barrier signal and paired MMA has landed.
  tc_fence_before_sync();
  __syncwarp();  // reconverge the role branches before the warp-aligned cluster barrier
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<2>(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && abort_flag != 0 && p.status != nullptr) atomicExch(p.status, int(ST_WAIT_TIMEOUT));
}

// ------------------------------------------------------------------ host side
namespace {

template <typename OutT, bool kBmn, int kMB, bool kFwd, bool kSK = false>
int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const DstMaps& dst, const GemmParams& p, int pairs,
                cudaStream_t stream) {
  using Cfg = PairCfg<kMB, kFwd>;
  auto kern = gemm_pair_kernel<OutT, kBmn, kMB, kFwd, kSK>;
  SX_ENSURE_DYN_SMEM(kern, Cfg::DYN_SMEM);
  // Row-sharded launches order themselves with flags in peer memory and are left out of the programmatic overlap.
  const bool pdl = !kFwd && p.n_dst <= 1 && pdl_enabled();
  return launch_kernel_ex(kern, 2u * (unsigned)pairs, Cfg::THREADS, Cfg::DYN_SMEM, stream, 2, pdl, tmA, tmB, dst, p) ==
                 cudaSuccess
             ? SX_OK
             : SX_ERR_EXEC;
}

template <typename OutT, bool kBmn>
int launch_pair_mb(int mb, const CUtensorMap& tmA, const CUtensorMap& tmB, const DstMaps& dst, const GemmParams& p,
                   int pairs, cudaStream_t stream) {
  if (p.sk_ws != nullptr) return launch_pair<OutT, kBmn, 2, false, true>(tmA, tmB, dst, p, pairs, stream);
  if (p.xchg >= XCHG_FORWARD)
    return mb == 2 ? launch_pair<OutT, kBmn, 2, true>(tmA, tmB, dst, p, pairs, stream)
                   : launch_pair<OutT, kBmn, 1, true>(tmA, tmB, dst, p, pairs, stream);
  return mb == 2 ? launch_pair<OutT, kBmn, 2, false>(tmA, tmB, dst, p, pairs, stream)
                 : launch_pair<OutT, kBmn, 1, false>(tmA, tmB, dst, p, pairs, stream);
}

}  // namespace

// bf16 operands only (a.kind == 0); operand conventions of launch_gemm_tc. a.bn selects the pair tile:
// 512 -> 512 x 256 (256 rows per CTA), anything else -> 256 x 256.
int launch_gemm_pair(const TcGemmArgs& a, cudaStream_t stream) {
  if (a.kind != 0 || a.nseg != 1) return SX_ERR_INVALID;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) return SX_ERR_INVALID;
  if ((a.lda * 2) % 16 || (a.ldb * 2) % 16 || (a.a_plane_stride * 2) % 16 || (a.b_plane_stride * 2) % 16)
    return SX_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(a.A) % 16 || reinterpret_cast<uintptr_t>(a.B) % 16) return SX_ERR_INVALID;
  const int mb = a.bn == 512 ? 2 : 1;
  const int bm = 256 * mb;

  CUtensorMap tmA, tmB;
  {
    uint64_t dims[3] = {(uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.za};
    uint64_t strides[2] = {(uint64_t)a.lda * 2, (uint64_t)a.a_plane_stride * 2};
    uint32_t box[3] = {64u, (uint32_t)(128 * mb), 1u};
    int rc = encode_tensor_map_3d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.A, dims, strides, box);
    if (rc != SX_OK) return rc;
  }
  if (a.b_mn) {
    uint64_t dims[3] = {(uint64_t)a.N, (uint64_t)a.K, (uint64_t)a.zb};
    uint64_t strides[2] = {(uint64_t)a.ldb * 2, (uint64_t)a.b_plane_stride * 2};
    uint32_t box[3] = {64u, 64u, 1u};
    int rc = encode_tensor_map_3d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.B, dims, strides, box);
    if (rc != SX_OK) return rc;
  } else {
    uint64_t dims[3] = {(uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.zb};
    uint64_t strides[2] = {(uint64_t)a.ldb * 2, (uint64_t)a.b_plane_stride * 2};
    uint32_t box[3] = {64u, 128u, 1u};
    int rc = encode_tensor_map_3d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.B, dims, strides, box);
    if (rc != SX_OK) return rc;
  }

  GemmParams p{};
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.batch = a.batch;
  p.nseg = 1;
  p.a_planes = 1; p.b_planes = 1;
  p.C = a.C; p.ldc = a.ldc; p.c_batch_stride = a.c_batch_stride;
  p.bias = a.bias; p.residual = a.residual;
  p.alpha = a.alpha; p.beta = a.beta; p.act = a.act;
  p.status = a.status;
  p.m_tiles = (int)((a.M + bm - 1) / bm);
  p.n_tiles = (int)((a.N + 255) / 256);
  p.group_m = a.group_m > 0 ? a.group_m : (mb == 2 ? 4 : 8);

  // Output path. Staged TMA stores need 16-byte aligned rows; they are what carries C to peer GPUs, and they
  // also replace 32 scattered 16-byte stores per warp instruction by one bulk store per 32 x 128-byte block.
  static DstMaps dst;  // zero-initialised maps are never dereferenced when n_dst == 0
  DstMaps dmaps = dst;
  const int out_elt = a.out_bf16 ? 2 : 4;
  const bool c_tma_ok = (a.ldc * out_elt) % 16 == 0 && (a.c_batch_stride * out_elt) % 16 == 0 &&
                        reinterpret_cast<uintptr_t>(a.C) % 16 == 0;
  p.n_dst = 0;
  p.wait_limit_ns = a.wait_limit_ns ? a.wait_limit_ns : WAIT_LIMIT_NS;
  if (a.n_peers > 0 && !c_tma_ok) return SX_ERR_INVALID;
  if (a.n_peers < 0 || a.n_peers > MAX_DST - 1) return SX_ERR_INVALID;
  p.xchg = a.n_peers > 0 ? (a.xchg ? a.xchg : XCHG_EPILOGUE_TMA) : XCHG_NONE;
  const bool fwd = p.xchg >= XCHG_FORWARD;
  if (fwd) {
    // The forwarders address C by bytes: one batch entry, flags and the completion counter are required.
    if (a.batch != 1 || a.flags == nullptr || a.xchg_counter == nullptr || a.epoch == 0) return SX_ERR_INVALID;
    if (p.xchg == XCHG_MULTICAST && (a.mc_C == nullptr || reinterpret_cast<uintptr_t>(a.mc_C) % 16)) return SX_ERR_INVALID;
    p.n_peers = a.n_peers;
    p.my_rank = a.my_rank;
    for (int i = 0; i < a.n_peers; ++i) {
      if (a.peer_flags[i] == nullptr || a.peer_rank[i] < 0 || a.peer_rank[i] >= 8) return SX_ERR_INVALID;
      if (p.xchg == XCHG_FORWARD && (a.peer_C[i] == nullptr || reinterpret_cast<uintptr_t>(a.peer_C[i]) % 16))
        return SX_ERR_INVALID;
      p.peer_rank[i] = a.peer_rank[i];
      p.peer_C[i] = const_cast<void*>(a.peer_C[i]);
      p.peer_flags[i] = a.peer_flags[i];
    }
    p.mc_C = a.mc_C;
    p.flags = a.flags;
    p.epoch = a.epoch;
    p.xchg_counter = a.xchg_counter;
  }
  const int n_maps = fwd ? 0 : a.n_peers;  // tensor maps of peer buffers are needed by the TMA forwarding only
  if (c_tma_ok && (a.tma_store || a.n_peers > 0)) {
    const CUtensorMapDataType odt = a.out_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    uint64_t dims[3] = {(uint64_t)a.N, (uint64_t)a.M, (uint64_t)a.batch};
    uint64_t strides[2] = {(uint64_t)a.ldc * out_elt, (uint64_t)a.c_batch_stride * out_elt};
    uint32_t box[3] = {(uint32_t)(128 / out_elt), 32u, 1u};
    for (int i = 0; i <= n_maps; ++i) {
      const void* base = i == 0 ? a.C : a.peer_C[i - 1];
      if (base == nullptr || reinterpret_cast<uintptr_t>(base) % 16) return SX_ERR_INVALID;
      int rc = encode_tensor_map_3d(&dmaps.m[i], odt, base, dims, strides, box);
      if (rc != SX_OK) return rc;
    }
    p.n_dst = 1 + n_maps;
  }
  const long long total = (long long)p.batch * p.m_tiles * p.n_tiles;
  const int max_pairs = a.num_sms / 2;
  int pairs = (int)(total < max_pairs ? total : max_pairs);
  if (a.sk_ws != nullptr) {
    // Stream-K: every pair of the device takes an equal range of k-blocks. Each range must be long enough to hold
    // the grain it is rounded to, or a pair would be left without work and the owner of its tile would wait for it.
    const long long nkb = (a.K + 63) / 64;
    if (mb != 2 || a.n_peers > 0 || a.sk_flags == nullptr || a.sk_epoch == 0 || total * nkb < (long long)max_pairs * 2 * SK_GRAIN ||
        total * nkb > 0x7fffffffLL || reinterpret_cast<uintptr_t>(a.sk_ws) % 16)
      return SX_ERR_INVALID;
    p.sk_ws = a.sk_ws;
    p.sk_flags = a.sk_flags;
    p.sk_epoch = a.sk_epoch;
    pairs = max_pairs;
  }
  if (a.out_bf16)
    return a.b_mn ? launch_pair_mb<__nv_bfloat16, true>(mb, tmA, tmB, dmaps, p, pairs, stream)
                  : launch_pair_mb<__nv_bfloat16, false>(mb, tmA, tmB, dmaps, p, pairs, stream);
  return a.b_mn ? launch_pair_mb<float, true>(mb, tmA, tmB, dmaps, p, pairs, stream)
                : launch_pair_mb<float, false>(mb, tmA, tmB, dmaps, p, pairs, stream);
}


// The work list of one CTA pair, produced on the host by the iterator the kernel's roles run (for tests): up to `cap`
// items of {tile, first k-block, end k-block, kind}; returns how many the pair has.
int stream_k_work_items(int pair, int pairs, int tiles, int nkb, int* out, int cap) {
  int n = 0;
  for (PairWork<true> w(pair, pairs, tiles, nkb); w.valid(); w.next(), ++n) {
    if (out != nullptr && n < cap) {
      out[4 * n + 0] = w.t;
      out[4 * n + 1] = w.kb0;
      out[4 * n + 2] = w.kb1;
      out[4 * n + 3] = w.kind;
    }
  }
  return n;
}
// Pairs whose partial sums the owner of `tile` adds (the count the epilogue computes): pairs below `pair` whose range
// reaches into the tile.
int stream_k_contributors(int pair, int pairs, int tiles, int nkb, int tile) {
  const long long total = (long long)tiles * nkb, tile_u0 = (long long)tile * nkb;
  int n = 0;
  for (int q = pair - 1; q >= 0 && sk_start(total, pairs, q + 1) > tile_u0; --q) ++n;
  return n;
}

size_t stream_k_workspace_bytes(int num_sms) { return (size_t)(num_sms / 2) * 512 * 256 * sizeof(float); }
int stream_k_flag_words(int num_sms) { return (num_sms / 2) * 2 * PairCfg<2>::EPI_WARPS; }

KernelShape describe_gemm_pair(int kmb) {
  auto mk = [](auto cfg) {
    using C = decltype(cfg);
    // cta_group::2: one instruction spans both CTAs, 256 rows x 256 columns x 16
    return KernelShape{"gemm_pair_kernel", C::BM, C::BN, C::BK, 256, C::BN, C::UMMA_K, C::THREADS, 2, C::STAGES, C::DYN_SMEM, C::TMEM_COLS};
  };
  return kmb == 2 ? mk(PairCfg<2>{}) : mk(PairCfg<1>{});
}

}  // namespace sx
