// Parameter block shared by the tcgen05 GEMM kernels and their host launchers.
#pragma once
#include <stdint.h>

namespace sx {

enum Activation : int {
  ACT_NONE = 0,
  ACT_RELU = 1,
  ACT_GELU = 2,  // tanh form: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
  ACT_SIGMOID = 3,
  ACT_TANH = 4,
  ACT_SILU = 5,
};

enum KernelStatus : int {
  ST_OK = 0,
  ST_WAIT_TIMEOUT = 5,  // a bounded mbarrier wait ran out; the kernel unwound and returned
};

// One launch computes, for every z in [0, batch):
//   C_z = act(alpha * sum_s A[z*a_planes + a_plane[s]] . B[z*b_planes + b_plane[s]] + beta * R_z + bias)
// nseg = 1 is a plain GEMM; nseg = 3 with planes (hi,hi), (hi,lo), (lo,hi) is the 3xTF32 product.
struct GemmParams {
  int M, N, K;
  int batch;
  int nseg;
  int a_plane[3];
  int b_plane[3];
  int a_planes, b_planes;
  void* C;
  long long ldc;             // elements
  long long c_batch_stride;  // elements
  const float* bias;         // fp32[N], broadcast over rows; may be null
  const void* residual;      // same dtype/layout as C; may be null (beta ignored then)
  float alpha, beta;
  int act;
  int* status;  // device word, receives KernelStatus on failure
  int m_tiles, n_tiles, group_m;
  int n_dst;  // 0: epilogue stores straight from registers; >= 1: staged in shared memory and written by TMA
              // to n_dst destinations (the local C first, then the same tile of every peer GPU's C)
  // Exchange of a row-sharded product with the other GPUs of the box (pair kernels only; see Exchange below).
  int xchg;                // Exchange mode
  int n_peers;             // other ranks (<= 7)
  int my_rank;
  int peer_rank[7];        // rank of peer j
  void* peer_C[7];         // peer j's copy of the region C points at, mapped into this process
  void* mc_C;              // multicast mapping of that region (XCHG_MULTICAST)
  int* flags;              // this rank's flag block (FLAG_WORDS ints, written by the peers)
  int* peer_flags[7];      // peer j's flag block, mapped into this process
  int epoch;               // collective call number (> 0, the same on every rank)
  unsigned* xchg_counter;  // device word of this GPU, zero between launches: forwarder warps that have finished
  unsigned long long wait_limit_ns;  // bound of every device-side wait of this launch
  int fault_stop_early;    // self-test only: the TMA producer leaves out the last k-block of the first tile
  // Stream-K (512 x 256 pair kernel, sk_ws != null): the k-blocks of all tiles are cut into one equal range per CTA
  // pair; a pair that works on a part of a tile without its last k-block leaves its partial sums in its slot of
  // sk_ws and raises its words of sk_flags to sk_epoch, the pair with the tile's last k-block adds them.
  float* sk_ws;            // one slot of 512 x 256 floats per CTA pair of the grid
  int* sk_flags;           // 16 words per CTA pair (2 CTAs x 8 epilogue warps), never reset: compared with sk_epoch
  int sk_epoch;            // number of this launch among the stream-K launches of the device (!= 0)
};

// How the tiles of a row-sharded product reach the other GPUs.
enum Exchange : int {
  XCHG_NONE = 0,
  XCHG_EPILOGUE_TMA = 1,  // each epilogue warp reads its blocks back from the local C (L2) by TMA and TMA-stores them
                          // to every peer (n_dst - 1 tensor maps); the caller orders the ranks
  XCHG_FORWARD = 2,       // dedicated forwarder warps copy finished tiles from the local C to every peer with
                          // 16-byte loads and stores; ranks are ordered by flags inside the kernel
  XCHG_MULTICAST = 3,     // the same warps store each 16 bytes once, to the multicast mapping (multimem.st): the
                          // NVSwitch delivers it to every GPU of the group
};

// Layout of a flag block: READY[r] = rank r has entered collective call `epoch` (everything it did with the previous
// C is complete, its C may be overwritten); DONE[r] = all of rank r's tiles of call `epoch` have landed here.
constexpr int FLAG_READY = 0;
constexpr int FLAG_DONE = 8;
constexpr int FLAG_WORDS = 16;

// Tensor maps of the output destinations of the TMA-store epilogue (local C, then peers' C).
constexpr int MAX_DST = 8;

}  // namespace sx
