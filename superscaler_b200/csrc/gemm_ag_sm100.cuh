// Communication arguments of the fused all-gather + GEMM kernel (gemm_ag_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_sm100.cuh"

namespace ssb {

struct GemmAgComm {
  const void* x_local;            // this rank's rows [M / tp][K] bf16, dense
  void* const* gather_ptrs;       // device array [tp]: every rank's gather buffer [M][K] bf16 (this call's parity)
  const void* gather_ptrs_host_local;  // this rank's gather buffer (host copy of gather_ptrs[rank], for the tensor map)
  uint32_t* const* flag_ptrs;     // device array [tp]: every rank's flag table, one word per 128-row block of M
  int rank, tp;
  uint32_t epoch;                 // grows by 1 per call on every rank
  int max_blocks;                 // capacity of the flag table
  long long capacity_elems;       // elements in a gather buffer
};

int gemm_ag_launch(const void* W, int ldw, const GemmParams& p, const GemmAgComm& cm, int num_sms, cudaStream_t stream);

}  // namespace ssb
