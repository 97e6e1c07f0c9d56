// Parameters of the tcgen05 GEMM family (host + device view).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ssb {

enum GemmAct : int {
  kActNone = 0,
  kActGelu = 1,    // v = gelu_tanh(v)
  kActRelu = 2,    // v = max(v, 0)
  kActDGelu = 3,   // v = v * gelu_tanh'(aux)          (aux = saved pre-activation)
  kActDRelu = 4,   // v = aux > 0 ? v : 0
};

// D[M,N] = epilogue( alpha * sum_k A[m,k] * B[n,k] )
//
// Operand storage (bf16, row-major, leading dimension in elements, multiple of 8):
//   a_mn_major = 0: A is stored [M][K]   (K contiguous);   1: A is stored [K][M]
//   b_mn_major = 0: B is stored [N][K]   (K contiguous);   1: B is stored [K][N]
// so forward  Y = X W^T       is (0,0) with A = X[M,K],  B = W[N,K];
//    dgrad    dX = dY W       is (0,1) with A = dY[M,N], B = W stored [N][K] = [K'][N'];
//    wgrad    dW = dY^T X     is (1,1) with A = dY stored [M][N] = [K'][M'], B = X stored [K'][N'].
//
// Epilogue, in this order, per element v (fp32):
//   v *= alpha; v += bias[n]; preact_out[m,n] = bf16(v); v = act(v) (aux for the derivative forms);
//   dropout (v = keep ? v / keep_prob : 0); v += residual[m,n]; if (accumulate) v += D[m,n]; store.
struct GemmParams {
  int M, N, K;
  void* D;
  int ldd;
  int out_fp32;
  int accumulate;
  float alpha;
  const void* bias;
  int bias_fp32;
  int act;
  const void* aux;  // bf16 [M, ldaux]
  int ldaux;
  void* preact_out;  // bf16 [M, ldpre] or null
  int ldpre;
  const void* residual;  // bf16 [M, ldres] or null
  int ldres;
  float dropout_p;         // 0 = off
  unsigned long long dropout_seed;
  int* status;             // device int, set to a StatusCode on failure (never cleared by the kernel)
  // Split-K (one-CTA kernel, plain fp32 outputs only): k_splits > 1 divides the reduction into that many slices,
  // each slice writes its [M, N] partial product into split_ws[slice] and a second kernel adds the slices in order
  // into D.  0 or 1 = off.  gemm_splitk_splits() says when it pays.
  int k_splits;
  float* split_ws;
};

// Number of reduction slices gemm_bf16_launch would like for this problem (1 = none): small outputs with a long
// reduction (weight gradients of narrow layers over many tokens or pixels) otherwise leave most SMs idle.
int gemm_splitk_splits(int M, int N, int K, int num_sms);

}  // namespace ssb
