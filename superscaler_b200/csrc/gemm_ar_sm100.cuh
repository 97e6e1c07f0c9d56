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
};

// Size (in 32-bit words) of one rank's flag table for `max_tiles` output tiles of 128 x 256.
inline long long gemm_ar_flag_words(int max_tiles, int tp) { return static_cast<long long>(max_tiles) * (tp * 4 + 4); }

int gemm_ar_launch(const void* A, int lda, const void* B, int ldb, int b_mn_major, const GemmParams& p,
                   const GemmArComm& cm, int num_sms, cudaStream_t stream);

}  // namespace ssb
