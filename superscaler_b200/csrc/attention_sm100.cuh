// Parameters of the tcgen05 flash-attention kernels (forward, dK/dV backward, dQ backward).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ssb {

// All activations are 2-D row-major bf16 matrices whose rows are tokens in batch-major order
// (row = b * S + s) and whose columns hold the heads side by side; `*_col0` is the first column of
// head 0 inside the matrix and `ld*` its row stride in elements, so Q, K and V can be three column
// ranges of one fused QKV GEMM output.
struct AttnParams {
  int B, NH, SQ, SK, HD;
  int q_col0, k_col0, v_col0;
  float scale;            // logits are scale * q.k
  int causal;             // 1: key index <= query index (requires SQ == SK)
  const int* kv_lens;     // optional [B]: keys >= kv_lens[b] are masked (padding mask)
  float dropout_p;
  unsigned long long dropout_seed;
  // forward outputs / backward inputs
  void* O;  int ldo; int o_col0;     // bf16 [B*SQ, ldo]
  float* LSE;                        // [B, NH, SQ]  log-sum-exp of the scaled logits (natural log)
  // backward only
  const float* delta;                // [B, NH, SQ]  rowsum(dO * O)
  void* dQ; int lddq; int dq_col0;
  void* dK; int lddk; int dk_col0;
  void* dV; int lddv; int dv_col0;
  int* status;
  // Optional additive bias on the scores that depends on (head, key - query) only (relative-position bias):
  // logits are scale * q.k + bias_table[head][key - query + SQ - 1]; fp32 [NH][SQ + SK - 1].  dbias_table, same
  // shape, receives (accumulates) its gradient in the fused backward kernel.  Null: no bias.
  const float* bias_table;
  float* dbias_table;
};

}  // namespace ssb
