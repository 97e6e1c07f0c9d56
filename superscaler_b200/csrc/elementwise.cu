// Stand-alone elementwise kernels for ops that are not absorbed by a GEMM epilogue
// (an op can sit alone in a pipeline stage, so each one must also exist by itself):
//   bias + GeLU fwd / bwd           (reference: runtime/megatron/model/fused_bias_gelu.py:31-45)
//   residual + dropout(x + bias)    (reference: runtime/megatron/model/flex_ops.py:61-83)
//   dropout fwd / bwd, ReLU fwd / bwd, add.
// All kernels stream 16 bytes per thread per access; rows are [rows, N] bf16, N % 8 == 0.
#include "common.cuh"

namespace ssb {
namespace {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]); q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]); q.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = q;
}

enum EwOp : int {
  kEwBiasGelu = 0,      // out = gelu(x + bias)
  kEwBiasGeluBwd = 1,   // out = g * gelu'(x + bias)         (x = saved input, a = g)
  kEwBiasDropAdd = 2,   // out = residual + dropout(x + bias)
  kEwDropout = 3,       // out = dropout(x)
  kEwDropoutBwd = 4,    // out = mask * g / keep             (x = g)
  kEwRelu = 5,          // out = max(x + bias, 0)
  kEwReluBwd = 6,       // out = (x + bias) > 0 ? g : 0      (x = saved input, a = g)
  kEwAdd = 7,           // out = x + a
};

template <int OP>
__global__ void __launch_bounds__(256)
ew_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ a,
          const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, long long nvec, int N,
          float dropout_p, unsigned long long seed) {
  const uint32_t keep16 = dropout_keep16(dropout_p);
  const float scale = 65536.0f / static_cast<float>(keep16);
  const int nvec_row = N / 8;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    float f[8], g[8], b[8];
    load8(x + v * 8, f);
    if (OP == kEwBiasGeluBwd || OP == kEwBiasDropAdd || OP == kEwReluBwd || OP == kEwAdd) load8(a + v * 8, g);
    const bool has_bias = bias != nullptr;
    if (has_bias && (OP == kEwBiasGelu || OP == kEwBiasGeluBwd || OP == kEwBiasDropAdd || OP == kEwRelu ||
                     OP == kEwReluBwd)) {
      load8(bias + (v % nvec_row) * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += b[j];
    }
    float o[8];
    if (OP == kEwBiasGelu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = gelu_tanh(f[j]);
    } else if (OP == kEwBiasGeluBwd) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = g[j] * gelu_tanh_grad(f[j]);
    } else if (OP == kEwRelu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = fmaxf(f[j], 0.f);
    } else if (OP == kEwReluBwd) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = f[j] > 0.f ? g[j] : 0.f;
    } else if (OP == kEwAdd) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = f[j] + g[j];
    } else {
      // dropout family: element index = v*8 + j, hash groups of 4
      uint32_t m0 = 0xF, m1 = 0xF;
      if (dropout_p > 0.f) {
        m0 = dropout_keep4(seed, static_cast<uint64_t>(v) * 2, keep16);
        m1 = dropout_keep4(seed, static_cast<uint64_t>(v) * 2 + 1, keep16);
      }
      const float sc = dropout_p > 0.f ? scale : 1.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[j] = ((m0 >> j) & 1u) ? f[j] * sc : 0.f;
        o[4 + j] = ((m1 >> j) & 1u) ? f[4 + j] * sc : 0.f;
      }
      if (OP == kEwBiasDropAdd) {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += g[j];
      }
    }
    store8(out + v * 8, o);
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n) {
  for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    if (i + 4 <= n) {
      const float4 f = *reinterpret_cast<const float4*>(in + i);
      uint2 q;
      q.x = pack_bf16x2(f.x, f.y);
      q.y = pack_bf16x2(f.z, f.w);
      *reinterpret_cast<uint2*>(out + i) = q;
    } else {
      for (long long j = i; j < n; ++j) out[j] = __float2bfloat16(in[j]);
    }
  }
}

}  // namespace

// op: see EwOp.  x, a, out: [rows, N] bf16 contiguous; bias: [N] bf16 or null.
int elementwise_launch(int op, const void* x, const void* a, const void* bias, void* out, long long rows, int N,
                       float dropout_p, unsigned long long seed, int num_sms, cudaStream_t stream) {
  if (N % 8) return -3;
  const long long nvec = rows * (N / 8);
  long long want = (nvec + 255) / 256;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > num_sms * 32LL ? num_sms * 32LL : want));
  const auto* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  const auto* ab = reinterpret_cast<const __nv_bfloat16*>(a);
  const auto* bb = reinterpret_cast<const __nv_bfloat16*>(bias);
  auto* ob = reinterpret_cast<__nv_bfloat16*>(out);
#define SSB_EW(OP) ew_kernel<OP><<<blocks, 256, 0, stream>>>(xb, ab, bb, ob, nvec, N, dropout_p, seed)
  switch (op) {
    case kEwBiasGelu: SSB_EW(kEwBiasGelu); break;
    case kEwBiasGeluBwd: SSB_EW(kEwBiasGeluBwd); break;
    case kEwBiasDropAdd: SSB_EW(kEwBiasDropAdd); break;
    case kEwDropout: SSB_EW(kEwDropout); break;
    case kEwDropoutBwd: SSB_EW(kEwDropoutBwd); break;
    case kEwRelu: SSB_EW(kEwRelu); break;
    case kEwReluBwd: SSB_EW(kEwReluBwd); break;
    case kEwAdd: SSB_EW(kEwAdd); break;
    default: return -2;
  }
#undef SSB_EW
  return static_cast<int>(cudaGetLastError());
}

int cast_f32_to_bf16_launch(const float* in, void* out, long long n, int num_sms, cudaStream_t stream) {
  long long want = (n / 4 + 255) / 256;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > num_sms * 32LL ? num_sms * 32LL : want));
  cast_f32_to_bf16_kernel<<<blocks, 256, 0, stream>>>(in, reinterpret_cast<__nv_bfloat16*>(out), n);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ssb
