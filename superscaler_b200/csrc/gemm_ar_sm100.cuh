// Communication arguments of the fused GEMM + tensor-parallel all-reduce kernel (gemm_ar_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_sm100.cuh"

namespace ssb {

struct GemmArComm {
  // device arrays [tp] with every rank's address of the same symmetric buffer:
  const void* const* partial_ptrs;  // bf16 [tp source ranks][tiles / tp][4 quarters][8 chunks][32 rows][32 cols]: partial tiles pushed by every rank
  const void* const* result_ptrs;   // bf16 [tiles][128 x 256]: final tiles pushed by their owners (this call's parity)
  uint32_t* const* flag_ptrs;       // flag table
  int rank, tp;
  uint32_t epoch;                   // grows by 1 per call on every rank
  int max_tiles;                    // capacity of the flag table (tiles)
  long long capacity_elems;         // elements in each of the partial / result buffers
  int grid;                         // filled by the launcher: CTAs of the launch (equal on all ranks)
  // Reduce-scatter form (scatter = 1): rank r ends with rows [r * M / tp, (r + 1) * M / tp) of the reduced product in
  // its LOCAL output [M / tp][N] (p.D, p.residual describe those rows); nothing is pushed back to the peers.  M / tp
  // must be a multiple of 128.  Because no final tiles travel, nothing tells a rank that an owner has finished
  // reading the partials it pushed; instead every rank publishes "consumed" once per reduce-scatter call, and every
  // later call (of either form) waits for the consumed flags of `wait_consumed_epoch`, the epoch of the last
  // reduce-scatter call (0: none), before it overwrites the owner's scratch.
  int scatter;
  uint32_t wait_consumed_epoch;
};

// Size (in 32-bit words) of one rank's flag table for `max_tiles` output tiles of 128 x 256.
// Layout: [max_tiles][tp][4] partial-quarter flags, [max_tiles][4] final-quarter flags, [tp] consumed flags, one
// counter of this rank's CTAs that finished consuming.
inline long long gemm_ar_flag_words(int max_tiles, int tp) {
  return static_cast<long long>(max_tiles) * (tp * 4 + 4) + tp + 1;
}

int gemm_ar_launch(const void* A, int lda, const void* B, int ldb, int b_mn_major, const GemmParams& p,
                   const GemmArComm& cm, int num_sms, cudaStream_t stream);

}  // namespace ssb
