// Embedding and vocab-parallel cross-entropy kernels.
//
// embedding fwd : out[t,:] = dropout( W[id[t]-v0,:] (0 if id outside [v0,v1)) + P[pos[t],:] )
//                 (reference: runtime/megatron/mpu/layers.py:185-205 masked lookup,
//                  runtime/megatron/model/flex_ops.py:356-376 position add + dropout)
// embedding bwd : dW[id-v0,:] += g, dP[pos,:] += g with fp32 atomics into the main-grad buffers.
// cross entropy : two phases so that a tensor-parallel group can all-reduce the row statistics
//                 between them (reference: runtime/megatron/mpu/cross_entropy.py:36-115):
//   stats    : per row local max, sum exp(x - local max), and the target logit if it is local
//   finalize : loss = log(sum) + max - target; logits overwritten in place by
//              (softmax - onehot) * grad_scale  (the backward of the mean loss)
// One CTA per row; rows are V_local bf16 logits.
#include "common.cuh"

namespace ssb {
namespace {

__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const long long* __restrict__ pos,
                     const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ P,
                     __nv_bfloat16* __restrict__ out, long long tokens, int H, long long v0, long long v1,
                     float dropout_p, unsigned long long seed) {
  const uint32_t keep16 = dropout_keep16(dropout_p);
  const float scale = dropout_p > 0.f ? 65536.0f / static_cast<float>(keep16) : 1.0f;
  const int nvec = H / 8;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < tokens * nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = v / nvec;
    const int c = static_cast<int>(v % nvec);
    const long long id = ids[t];
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (id >= v0 && id < v1) {
      const uint4 q = *reinterpret_cast<const uint4*>(W + (id - v0) * H + c * 8);
      float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), cc = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = cc.x; f[5] = cc.y; f[6] = d.x; f[7] = d.y;
    }
    if (P != nullptr) {
      const uint4 q = *reinterpret_cast<const uint4*>(P + pos[t] * H + c * 8);
      float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), cc = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
      f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y; f[4] += cc.x; f[5] += cc.y; f[6] += d.x; f[7] += d.y;
    }
    if (dropout_p > 0.f) {
      const uint32_t m0 = dropout_keep4(seed, static_cast<uint64_t>(v) * 2, keep16);
      const uint32_t m1 = dropout_keep4(seed, static_cast<uint64_t>(v) * 2 + 1, keep16);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        f[j] = ((m0 >> j) & 1u) ? f[j] * scale : 0.f;
        f[4 + j] = ((m1 >> j) & 1u) ? f[4 + j] * scale : 0.f;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
    o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(out + v * 8) = o;
  }
}

// g is the gradient w.r.t. the embedding OUTPUT (after dropout); the mask is regenerated here.
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ ids, const long long* __restrict__ pos,
                     const __nv_bfloat16* __restrict__ g, float* __restrict__ dW, float* __restrict__ dP,
                     long long tokens, int H, long long v0, long long v1, float dropout_p, unsigned long long seed) {
  const uint32_t keep16 = dropout_keep16(dropout_p);
  const float scale = dropout_p > 0.f ? 65536.0f / static_cast<float>(keep16) : 1.0f;
  const int nvec = H / 8;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < tokens * nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = v / nvec;
    const int c = static_cast<int>(v % nvec);
    const uint4 q = *reinterpret_cast<const uint4*>(g + v * 8);
    float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), cc = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
    float f[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, d.x, d.y};
    if (dropout_p > 0.f) {
      const uint32_t m0 = dropout_keep4(seed, static_cast<uint64_t>(v) * 2, keep16);
      const uint32_t m1 = dropout_keep4(seed, static_cast<uint64_t>(v) * 2 + 1, keep16);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        f[j] = ((m0 >> j) & 1u) ? f[j] * scale : 0.f;
        f[4 + j] = ((m1 >> j) & 1u) ? f[4 + j] * scale : 0.f;
      }
    }
    const long long id = ids[t];
    if (dW != nullptr && id >= v0 && id < v1) {
      float* dst = dW + (id - v0) * H + c * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(dst + j, f[j]);
    }
    if (dP != nullptr) {
      float* dst = dP + pos[t] * H + c * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(dst + j, f[j]);
    }
  }
}

// Order-independent variant of the scatter above: `keys` are the row indices (token ids, or positions) in
// ascending order and `order[p]` is the token that holds keys[p].  Block p works only if it is the first of its
// run of equal keys; it then sums the run's rows in the order given and adds the total to row keys[p] - k0 of dst
// with plain stores (no other block touches that row), so repeated runs give bitwise equal results.
__global__ void __launch_bounds__(256)
embedding_bwd_sorted_kernel(const long long* __restrict__ keys, const long long* __restrict__ order,
                            const __nv_bfloat16* __restrict__ g, float* __restrict__ dst, long long tokens, int H,
                            long long k0, long long k1, float dropout_p, unsigned long long seed) {
  const long long p = blockIdx.x;
  const long long key = keys[p];
  if (key < k0 || key >= k1) return;
  if (p > 0 && keys[p - 1] == key) return;
  const uint32_t keep16 = dropout_keep16(dropout_p);
  const float scale = dropout_p > 0.f ? 65536.0f / static_cast<float>(keep16) : 1.0f;
  const int nvec = H / 8;
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (long long j = p; j < tokens && keys[j] == key; ++j) {
      const long long v = order[j] * nvec + c;
      const uint4 q = *reinterpret_cast<const uint4*>(g + v * 8);
      float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), cc = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
      float f[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, d.x, d.y};
      if (dropout_p > 0.f) {
        const uint32_t m0 = dropout_keep4(seed, static_cast<uint64_t>(v) * 2, keep16);
        const uint32_t m1 = dropout_keep4(seed, static_cast<uint64_t>(v) * 2 + 1, keep16);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          f[i] = ((m0 >> i) & 1u) ? f[i] * scale : 0.f;
          f[4 + i] = ((m1 >> i) & 1u) ? f[4 + i] * scale : 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    float4* out = reinterpret_cast<float4*>(dst + (key - k0) * H + c * 8);
    float4 lo = out[0], hi = out[1];
    lo.x += acc[0]; lo.y += acc[1]; lo.z += acc[2]; lo.w += acc[3];
    hi.x += acc[4]; hi.y += acc[5]; hi.z += acc[6]; hi.w += acc[7];
    out[0] = lo;
    out[1] = hi;
  }
}

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sm) {
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();  // protects `sm` between successive calls
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  const int nw = blockDim.x >> 5;
  float t = (threadIdx.x & 31) < nw ? sm[threadIdx.x & 31] : (is_max ? -INFINITY : 0.f);
  return is_max ? warp_max(t) : warp_sum(t);
}

// stats[row] = {local max, sum exp(x - local max), target logit or 0}
__global__ void __launch_bounds__(256)
ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, int ld, const long long* __restrict__ targets,
                float* __restrict__ row_max, float* __restrict__ row_sum, float* __restrict__ row_tgt, int V,
                long long v0) {
  __shared__ float sm[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* x = logits + row * ld;
  const int nvec = V / 8;
  float mx = -INFINITY;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 q = reinterpret_cast<const uint4*>(x)[v];
    float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
    mx = fmaxf(mx, fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y)), fmaxf(fmaxf(c.x, c.y), fmaxf(d.x, d.y))));
  }
  for (int k = nvec * 8 + threadIdx.x; k < V; k += blockDim.x) mx = fmaxf(mx, __bfloat162float(x[k]));
  mx = block_reduce(mx, true, sm);
  float s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 q = reinterpret_cast<const uint4*>(x)[v];
    float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
    s += __expf(a.x - mx) + __expf(a.y - mx) + __expf(b.x - mx) + __expf(b.y - mx) + __expf(c.x - mx) +
         __expf(c.y - mx) + __expf(d.x - mx) + __expf(d.y - mx);
  }
  for (int k = nvec * 8 + threadIdx.x; k < V; k += blockDim.x) s += __expf(__bfloat162float(x[k]) - mx);
  s = block_reduce(s, false, sm);
  if (threadIdx.x == 0) {
    row_max[row] = mx;
    row_sum[row] = s;
    const long long t = targets[row] - v0;
    row_tgt[row] = (t >= 0 && t < V) ? __bfloat162float(x[t]) : 0.f;
  }
}

// gmax / gsum / gtgt are the group-reduced statistics (gsum already rescaled to gmax by the caller for
// tensor parallel runs; for a single rank they are the outputs of ce_stats_kernel).
// loss_mask: optional fp32 [rows] weights (0 drops the token); grad_scale multiplies the gradient.
__global__ void __launch_bounds__(256)
ce_finalize_kernel(__nv_bfloat16* __restrict__ logits, int ld, const long long* __restrict__ targets,
                   const float* __restrict__ gmax, const float* __restrict__ gsum, const float* __restrict__ gtgt,
                   const float* __restrict__ loss_mask, float* __restrict__ loss, int V, long long v0,
                   float grad_scale, int write_grad) {
  const long long row = blockIdx.x;
  __nv_bfloat16* x = logits + row * ld;
  const float mx = gmax[row], sum = gsum[row];
  const float w = loss_mask ? loss_mask[row] : 1.0f;
  if (threadIdx.x == 0) loss[row] = (logf(sum) + mx - gtgt[row]) * w;
  if (!write_grad) return;
  const float inv = 1.0f / sum;
  const float gs = grad_scale * w;
  const long long t = targets[row] - v0;
  const int nvec = V / 8;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 q = reinterpret_cast<const uint4*>(x)[v];
    float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
    float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float pr = __expf(f[j] - mx) * inv;
      if (static_cast<long long>(v) * 8 + j == t) pr -= 1.0f;
      f[j] = pr * gs;
    }
    uint4 o;
    o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
    o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
    reinterpret_cast<uint4*>(x)[v] = o;
  }
  for (int k = nvec * 8 + threadIdx.x; k < V; k += blockDim.x) {
    float pr = __expf(__bfloat162float(x[k]) - mx) * inv;
    if (k == t) pr -= 1.0f;
    x[k] = __float2bfloat16(pr * gs);
  }
}

}  // namespace

int embedding_fwd_launch(const long long* ids, const long long* pos, const void* W, const void* P, void* out,
                         long long tokens, int H, long long v0, long long v1, float dropout_p,
                         unsigned long long seed, int num_sms, cudaStream_t stream) {
  if (H % 8) return -3;
  long long want = (tokens * (H / 8) + 255) / 256;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > num_sms * 32LL ? num_sms * 32LL : want));
  embedding_fwd_kernel<<<blocks, 256, 0, stream>>>(ids, pos, reinterpret_cast<const __nv_bfloat16*>(W),
                                                   reinterpret_cast<const __nv_bfloat16*>(P),
                                                   reinterpret_cast<__nv_bfloat16*>(out), tokens, H, v0, v1,
                                                   dropout_p, seed);
  return static_cast<int>(cudaGetLastError());
}

int embedding_bwd_launch(const long long* ids, const long long* pos, const void* g, float* dW, float* dP,
                         long long tokens, int H, long long v0, long long v1, float dropout_p,
                         unsigned long long seed, int num_sms, cudaStream_t stream) {
  if (H % 8) return -3;
  long long want = (tokens * (H / 8) + 255) / 256;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > num_sms * 32LL ? num_sms * 32LL : want));
  embedding_bwd_kernel<<<blocks, 256, 0, stream>>>(ids, pos, reinterpret_cast<const __nv_bfloat16*>(g), dW, dP,
                                                   tokens, H, v0, v1, dropout_p, seed);
  return static_cast<int>(cudaGetLastError());
}

int embedding_bwd_sorted_launch(const long long* keys, const long long* order, const void* g, float* dst,
                                long long tokens, int H, long long k0, long long k1, float dropout_p,
                                unsigned long long seed, cudaStream_t stream) {
  if (H % 8) return -3;
  if (tokens < 1 || tokens > 0x7fffffffLL) return -4;
  embedding_bwd_sorted_kernel<<<static_cast<unsigned>(tokens), 256, 0, stream>>>(
      keys, order, reinterpret_cast<const __nv_bfloat16*>(g), dst, tokens, H, k0, k1, dropout_p, seed);
  return static_cast<int>(cudaGetLastError());
}

int ce_stats_launch(const void* logits, int ld, const long long* targets, float* row_max, float* row_sum,
                    float* row_tgt, long long rows, int V, long long v0, cudaStream_t stream) {
  if (ld % 8) return -3;
  ce_stats_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld,
                                                                   targets, row_max, row_sum, row_tgt, V, v0);
  return static_cast<int>(cudaGetLastError());
}

int ce_finalize_launch(void* logits, int ld, const long long* targets, const float* gmax, const float* gsum,
                       const float* gtgt, const float* loss_mask, float* loss, long long rows, int V, long long v0,
                       float grad_scale, int write_grad, cudaStream_t stream) {
  if (ld % 8) return -3;
  ce_finalize_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(logits), ld,
                                                                      targets, gmax, gsum, gtgt, loss_mask, loss, V,
                                                                      v0, grad_scale, write_grad);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ssb
