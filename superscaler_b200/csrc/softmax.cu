// Stand-alone scaled softmax family (used when the attention ops of a plan are not
// co-located and cannot run as one flash-attention kernel):
//   causal : softmax(scale * x) over k <= q, zero elsewhere          [batches, s, s]
//   masked : softmax(scale * x) with uint8 mask (1 = masked -> -10000)   [b, np, sq, sk], mask [b|1, 1, sq, sk]
//   plain  : softmax(scale * x)
// and the shared backward dx = scale * (g*y - y * sum(g*y)).
// Same contracts as the reference's three extensions
// (runtime/megatron/fused_kernels/scaled_upper_triang_masked_softmax.h:113-330,
//  runtime/megatron/fused_kernels/scaled_masked_softmax.h:98-423), without their
// sk <= 2048 / 4096 limits: one warp per row, fp32 math, rows re-read from L1/L2.
#include "common.cuh"

namespace ssb {
namespace {

constexpr int kSmWarps = 4;

// mode: 0 plain, 1 causal, 2 masked
__global__ void __launch_bounds__(kSmWarps * 32)
softmax_fwd_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ mask, __nv_bfloat16* __restrict__ y,
                   long long rows, int sq, int sk, int heads, int mask_batch_stride_is_zero, float scale, int mode) {
  const int lane = threadIdx.x & 31;
  const long long w0 = blockIdx.x * static_cast<long long>(kSmWarps) + (threadIdx.x >> 5);
  for (long long row = w0; row < rows; row += static_cast<long long>(gridDim.x) * kSmWarps) {
    const int q = static_cast<int>(row % sq);
    const __nv_bfloat16* xr = x + row * sk;
    __nv_bfloat16* yr = y + row * sk;
    const int limit = (mode == 1) ? (q + 1) : sk;
    const uint8_t* mr = nullptr;
    if (mode == 2) {
      const long long b = row / (static_cast<long long>(sq) * heads);
      mr = mask + ((mask_batch_stride_is_zero ? 0 : b) * sq + q) * sk;
    }
    float mx = -INFINITY;
    for (int k = lane; k < limit; k += 32) {
      float v = __bfloat162float(xr[k]) * scale;
      if (mr && mr[k]) v = -10000.0f;
      mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int k = lane; k < limit; k += 32) {
      float v = __bfloat162float(xr[k]) * scale;
      if (mr && mr[k]) v = -10000.0f;
      sum += __expf(v - mx);
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int k = lane; k < sk; k += 32) {
      float o = 0.f;
      if (k < limit) {
        float v = __bfloat162float(xr[k]) * scale;
        if (mr && mr[k]) v = -10000.0f;
        o = __expf(v - mx) * inv;
      }
      yr[k] = __float2bfloat16(o);
    }
  }
}

__global__ void __launch_bounds__(kSmWarps * 32)
softmax_bwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ dx, long long rows, int sk, float scale) {
  const int lane = threadIdx.x & 31;
  const long long w0 = blockIdx.x * static_cast<long long>(kSmWarps) + (threadIdx.x >> 5);
  for (long long row = w0; row < rows; row += static_cast<long long>(gridDim.x) * kSmWarps) {
    const __nv_bfloat16* gr = g + row * sk;
    const __nv_bfloat16* yr = y + row * sk;
    float dot = 0.f;
    for (int k = lane; k < sk; k += 32) dot += __bfloat162float(gr[k]) * __bfloat162float(yr[k]);
    dot = warp_sum(dot);
    for (int k = lane; k < sk; k += 32) {
      const float yy = __bfloat162float(yr[k]);
      dx[row * sk + k] = __float2bfloat16(scale * (__bfloat162float(gr[k]) * yy - yy * dot));
    }
  }
}

}  // namespace

int softmax_fwd_launch(const void* x, const void* mask, void* y, long long rows, int sq, int sk, int heads,
                       int mask_broadcast_batch, float scale, int mode, int num_sms, cudaStream_t stream) {
  long long want = (rows + kSmWarps - 1) / kSmWarps;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > num_sms * 16LL ? num_sms * 16LL : want));
  softmax_fwd_kernel<<<blocks, kSmWarps * 32, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const uint8_t*>(mask),
      reinterpret_cast<__nv_bfloat16*>(y), rows, sq, sk, heads, mask_broadcast_batch, scale, mode);
  return static_cast<int>(cudaGetLastError());
}

int softmax_bwd_launch(const void* g, const void* y, void* dx, long long rows, int sk, float scale, int num_sms,
                       cudaStream_t stream) {
  long long want = (rows + kSmWarps - 1) / kSmWarps;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > num_sms * 16LL ? num_sms * 16LL : want));
  softmax_bwd_kernel<<<blocks, kSmWarps * 32, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(g),
                                                           reinterpret_cast<const __nv_bfloat16*>(y),
                                                           reinterpret_cast<__nv_bfloat16*>(dx), rows, sk, scale);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ssb
