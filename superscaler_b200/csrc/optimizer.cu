// Fused optimizer kernels over FLAT buffers: every parameter of a pipeline stage lives in one
// contiguous fp32 master buffer, with matching fp32 gradient, Adam moment and bf16 model buffers.
// One launch replaces the reference's chain of apex multi-tensor kernels: copy model grads to main
// grads, unscale + inf check, l2 norm, clip, FusedAdam, copy main params back to half
// (runtime/megatron/optimizer/optimizer.py:348-390,404-443,
//  runtime/megatron/optimizer/clip_grads.py:29-120).
//
//   sumsq  : sum of squares of the gradient buffer (two-stage, deterministic)
//   adam   : p, m, v update with the clip coefficient and the inf/nan skip decided ON DEVICE from the
//            reduced sum of squares (no host synchronisation), bf16 copy-out of the new parameters,
//            optional zeroing of the gradient buffer for the next iteration.
//   sgd    : momentum SGD with the same plumbing (the reference uses apex FusedSGD for --optimizer sgd).
#include "common.cuh"

namespace ssb {
namespace {

__global__ void __launch_bounds__(256)
sumsq_partial_kernel(const float* __restrict__ g, long long n, float* __restrict__ partials) {
  __shared__ float sm[8];
  float s = 0.f;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 f = reinterpret_cast<const float4*>(g)[i];
    s += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const float f = g[n4 * 4 + threadIdx.x];
    s += f * f;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? sm[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) partials[blockIdx.x] = t;
  }
}

__global__ void sumsq_fold_kernel(const float* __restrict__ partials, int n, float* __restrict__ out, int accumulate) {
  __shared__ float sm[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partials[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? sm[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + t : t;
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay;
  float bias_corr1, bias_corr2;  // 1 - beta^t
  float grad_scale;              // gradients are multiplied by this first (1/num_microbatches, 1/loss_scale)
  float max_norm;                // <= 0: no clipping
  long long wd_end;              // elements [0, wd_end) get weight decay, the rest none
  int zero_grad;
};

__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, float* __restrict__ g,
            __nv_bfloat16* __restrict__ p16, long long n, const float* __restrict__ sumsq, int* __restrict__ skipped,
            AdamArgs a) {
  float clip = 1.0f;
  if (sumsq != nullptr) {
    const float ss = sumsq[0];
    if (!isfinite(ss)) {  // inf / nan gradients: leave the parameters alone, report, still clear the grads
      if (blockIdx.x == 0 && threadIdx.x == 0 && skipped != nullptr) atomicAdd(skipped, 1);
      if (a.zero_grad) {
        for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
             i += static_cast<long long>(gridDim.x) * blockDim.x)
          g[i] = 0.f;
      }
      return;
    }
    if (a.max_norm > 0.f) {
      const float norm = sqrtf(ss) * a.grad_scale;
      clip = fminf(1.0f, a.max_norm / (norm + 1.0e-6f));
    }
  }
  const float gs = a.grad_scale * clip;
  const float inv_bc1 = 1.0f / a.bias_corr1;
  const float inv_sqrt_bc2 = rsqrtf(a.bias_corr2);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float gi = g[i] * gs;
    const float mi = a.beta1 * m[i] + (1.0f - a.beta1) * gi;
    const float vi = a.beta2 * v[i] + (1.0f - a.beta2) * gi * gi;
    float pi = p[i];
    const float denom = sqrtf(vi) * inv_sqrt_bc2 + a.eps;
    const float wd = i < a.wd_end ? a.weight_decay : 0.f;
    pi -= a.lr * ((mi * inv_bc1) / denom + wd * pi);
    p[i] = pi;
    m[i] = mi;
    v[i] = vi;
    p16[i] = __float2bfloat16(pi);
    if (a.zero_grad) g[i] = 0.f;
  }
}

struct SgdArgs {
  float lr, momentum, weight_decay, grad_scale, max_norm;
  long long wd_end;
  int zero_grad, first_step;
};

__global__ void __launch_bounds__(256)
sgd_kernel(float* __restrict__ p, float* __restrict__ mom, float* __restrict__ g, __nv_bfloat16* __restrict__ p16,
           long long n, const float* __restrict__ sumsq, int* __restrict__ skipped, SgdArgs a) {
  float clip = 1.0f;
  if (sumsq != nullptr) {
    const float ss = sumsq[0];
    if (!isfinite(ss)) {
      if (blockIdx.x == 0 && threadIdx.x == 0 && skipped != nullptr) atomicAdd(skipped, 1);
      if (a.zero_grad)
        for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
             i += static_cast<long long>(gridDim.x) * blockDim.x)
          g[i] = 0.f;
      return;
    }
    if (a.max_norm > 0.f) clip = fminf(1.0f, a.max_norm / (sqrtf(ss) * a.grad_scale + 1.0e-6f));
  }
  const float gs = a.grad_scale * clip;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float pi = p[i];
    float gi = g[i] * gs + (i < a.wd_end ? a.weight_decay : 0.f) * pi;
    float bi = a.first_step ? gi : a.momentum * mom[i] + gi;
    mom[i] = bi;
    pi -= a.lr * bi;
    p[i] = pi;
    p16[i] = __float2bfloat16(pi);
    if (a.zero_grad) g[i] = 0.f;
  }
}

}  // namespace

constexpr int kSumsqBlocks = 1024;

// partials: scratch of kSumsqBlocks floats.  out[0] (+)= sum g^2.
int sumsq_launch(const float* g, long long n, float* partials, float* out, int accumulate, cudaStream_t stream) {
  long long want = (n / 4 + 255) / 256;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > kSumsqBlocks ? kSumsqBlocks : want));
  sumsq_partial_kernel<<<blocks, 256, 0, stream>>>(g, n, partials);
  sumsq_fold_kernel<<<1, 256, 0, stream>>>(partials, blocks, out, accumulate);
  return static_cast<int>(cudaGetLastError());
}

int adam_launch(float* p, float* m, float* v, float* g, void* p16, long long n, const float* sumsq, int* skipped,
                float lr, float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale,
                float max_norm, long long wd_end, int zero_grad, int num_sms, cudaStream_t stream) {
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias_corr1 = 1.0f - powf(beta1, static_cast<float>(step));
  a.bias_corr2 = 1.0f - powf(beta2, static_cast<float>(step));
  a.grad_scale = grad_scale; a.max_norm = max_norm; a.wd_end = wd_end; a.zero_grad = zero_grad;
  long long want = (n + 255) / 256;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > num_sms * 16LL ? num_sms * 16LL : want));
  adam_kernel<<<blocks, 256, 0, stream>>>(p, m, v, g, reinterpret_cast<__nv_bfloat16*>(p16), n, sumsq, skipped, a);
  return static_cast<int>(cudaGetLastError());
}

int sgd_launch(float* p, float* mom, float* g, void* p16, long long n, const float* sumsq, int* skipped, float lr,
               float momentum, float weight_decay, float grad_scale, float max_norm, long long wd_end, int zero_grad,
               int first_step, int num_sms, cudaStream_t stream) {
  SgdArgs a;
  a.lr = lr; a.momentum = momentum; a.weight_decay = weight_decay; a.grad_scale = grad_scale; a.max_norm = max_norm;
  a.wd_end = wd_end; a.zero_grad = zero_grad; a.first_step = first_step;
  long long want = (n + 255) / 256;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > num_sms * 16LL ? num_sms * 16LL : want));
  sgd_kernel<<<blocks, 256, 0, stream>>>(p, mom, g, reinterpret_cast<__nv_bfloat16*>(p16), n, sumsq, skipped, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ssb
