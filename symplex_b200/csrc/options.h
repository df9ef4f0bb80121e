// Process-wide tuning overrides of the library (symplex_b200_set_option / symplex_b200_get_option).
// Every field has a value that means "the library decides"; the dispatch code reads the fields, never the
// environment. Two of them can be preset from the environment, read once when the library is loaded:
// SYMPLEX_B200_TILE (tile_n) and SYMPLEX_B200_TRACE (trace).
#pragma once
#include <atomic>
#include <cstdint>

namespace sx {

struct Options {
  std::atomic<int64_t> tile_n{0};          // 0 auto; 64 / 128 / 256: tile width of the single-CTA bf16 and pre-split fp32 kernels
  std::atomic<int64_t> pair_mode{-1};      // -1 auto; 0 single-CTA tiles, 1 256x256 CTA pairs, 2 512x256 CTA pairs (bf16)
  std::atomic<int64_t> f32_fused{-1};      // -1 auto; 0 / 1: fp32 operands split in shared memory instead of by a pre-pass
  std::atomic<int64_t> f32_split_k{0};     // 0 auto; 1 / 2 / 4: CTAs per output tile of the in-kernel-split fp32 kernel
  std::atomic<int64_t> f32_tile_rows{0};   // 0 auto; 128: problems with at most 64 rows also take the 128-row kernel
  std::atomic<int64_t> stream_k{0};        // 1: the 512x256 CTA pairs share the k-blocks of all tiles evenly wherever that can run (bf16, pooled scratch)
  std::atomic<int64_t> group_m{0};         // 0 auto; tile rows per band of the pair kernels' tile order
  std::atomic<int64_t> tma_store{1};       // 1: epilogues stage C in shared memory and store it by TMA where C qualifies
  std::atomic<int64_t> pipeline_mb{96};    // host-buffer GEMMs: MB of A + C per row chunk of the copy/compute pipeline
  std::atomic<int64_t> pipeline{1};        // 0: host-buffer GEMMs never chunk
  std::atomic<int64_t> wait_limit_ms{2000};  // bound of every device-side wait of the bf16 kernels
  std::atomic<int64_t> pdl{1};             // 1: the tcgen05 GEMM kernels are launched as programmatic dependents of the kernel before them in the stream
  std::atomic<int64_t> trace{0};           // 1: one line per GEMM dispatch on stderr
  std::atomic<int64_t> stream_k_launches{0};  // statistic, not a setting: stream-K launches so far (may be set back to 0)
};

Options& options();

}  // namespace sx
