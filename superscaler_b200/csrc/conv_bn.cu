// Convolution support kernels and BatchNorm / pooling for the Wide-ResNet family (NHWC, bf16).
//
// Convolutions run as GEMMs on the tcgen05 kernel of gemm_sm100.cu:
//   1x1 stride 1 : the NHWC activation IS the [N*H*W, C] GEMM operand (no copy);
//   1x1 stride s : `subsample` gathers the strided pixels first;
//   k x k        : `im2col` writes the patch matrix [N*Ho*Wo, k*k*C] (tap-major, channel-minor), the
//                  filter is stored [Cout, k*k*C]; dgrad is a GEMM followed by `col2im` (gather form,
//                  no atomics), wgrad is the MN-major GEMM of the output gradient with the patch matrix.
// They replace cuDNN behind torch.nn.Conv2d / BatchNorm2d / MaxPool2d / AdaptiveAvgPool2d in the
// reference's ParallelConvOp ... ParallelAdapAvgPoolOp (runtime/megatron/model/flex_ops.py:1423-1719).
//
// BatchNorm uses batch statistics of the local micro-batch only (the reference does not synchronise
// them across data-parallel ranks either) with fp32 accumulation; ReLU and the residual add are fused
// into the normalisation pass.
#include "common.cuh"

namespace ssb {
namespace {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]); q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]); q.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = q;
}

struct ConvGeom {
  int N, H, W, C, KH, KW, stride, pad, Ho, Wo, Kpad;  // Kpad = row length of the patch matrix (>= KH*KW*C)
};

// cols[(n, ho, wo), (r, s, c)] = x[n, ho*stride + r - pad, wo*stride + s - pad, c]  (0 outside)
// C % 8 == 0: one thread moves 8 channels of one tap.  The small-C variant handles the 3-channel stem.
__global__ void __launch_bounds__(256)
im2col_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ cols, ConvGeom g) {
  // A block takes one row of the patch matrix (one output pixel) at a time: the pixel's coordinates are worked out
  // once per row, and a thread's element inside the row needs one 32-bit division (tap = e / cvec).
  const int cvec = g.C / 8;
  const int per_row = g.KH * g.KW * cvec;
  const int rows = g.N * g.Ho * g.Wo;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const int wo = row % g.Wo, t = row / g.Wo;
    const int ho = t % g.Ho, n = t / g.Ho;
    const int h0 = ho * g.stride - g.pad, w0 = wo * g.stride - g.pad;
    const __nv_bfloat16* xin = x + static_cast<long long>(n) * g.H * g.W * g.C;
    __nv_bfloat16* out = cols + static_cast<long long>(row) * g.Kpad;
    for (int e = threadIdx.x; e < per_row; e += 256) {
      const int tap = e / cvec, c8 = e - tap * cvec;
      const int r = tap / g.KW, s2 = tap - r * g.KW;
      const int h = h0 + r, w = w0 + s2;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h >= 0 && h < g.H && w >= 0 && w < g.W)
        v = *reinterpret_cast<const uint4*>(xin + (static_cast<long long>(h) * g.W + w) * g.C + c8 * 8);
      *reinterpret_cast<uint4*>(out + e * 8) = v;     // (r, s, c) is the order of e: the row is written front to back
    }
  }
}

__global__ void __launch_bounds__(256)
im2col_small_c_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ cols, ConvGeom g) {
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * g.Kpad;
  const int kreal = g.KH * g.KW * g.C;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / g.Kpad;
    const int k = static_cast<int>(i % g.Kpad);
    __nv_bfloat16 v = __float2bfloat16(0.f);
    if (k < kreal) {
      const int c = k % g.C, s = (k / g.C) % g.KW, r = k / (g.C * g.KW);
      const int wo = static_cast<int>(row % g.Wo);
      const int ho = static_cast<int>((row / g.Wo) % g.Ho);
      const int n = static_cast<int>(row / (static_cast<long long>(g.Wo) * g.Ho));
      const int h = ho * g.stride + r - g.pad, w = wo * g.stride + s - g.pad;
      if (h >= 0 && h < g.H && w >= 0 && w < g.W) v = x[((static_cast<long long>(n) * g.H + h) * g.W + w) * g.C + c];
    }
    cols[i] = v;
  }
}

// dx[n, h, w, c] = sum over taps (r, s) with (h + pad - r) % stride == 0 ... of dcols[(n, ho, wo), (r, s, c)]
__global__ void __launch_bounds__(256)
col2im_kernel(const __nv_bfloat16* __restrict__ dcols, __nv_bfloat16* __restrict__ dx, ConvGeom g) {
  // A block takes 256 / cvec input pixels at a time (one when a pixel has more than 256 channel groups); a thread
  // keeps its pixel lane and first channel group for the whole kernel, so the flat-index divisions happen once.
  const int cvec = g.C / 8;
  const int ppb = cvec >= 256 ? 1 : 256 / cvec;
  const int pl = threadIdx.x / cvec, c_first = threadIdx.x - pl * cvec;
  if (pl >= ppb) return;
  const int c_step = ppb == 1 ? 256 : cvec;            // one group per thread unless the pixel is wider than the block
  const int pixels = g.N * g.H * g.W;
  for (int pix = blockIdx.x * ppb + pl; pix < pixels; pix += gridDim.x * ppb) {
    const int w = pix % g.W, t = pix / g.W;
    const int h = t % g.H, n = t / g.H;
    for (int c8 = c_first; c8 < cvec; c8 += c_step) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < g.KH; ++r) {
        const int hn = h + g.pad - r;
        if (hn < 0 || hn % g.stride) continue;
        const int ho = hn / g.stride;
        if (ho >= g.Ho) continue;
        for (int s2 = 0; s2 < g.KW; ++s2) {
          const int wn = w + g.pad - s2;
          if (wn < 0 || wn % g.stride) continue;
          const int wo = wn / g.stride;
          if (wo >= g.Wo) continue;
          float f[8];
          ld8(dcols + ((static_cast<long long>(n) * g.Ho + ho) * g.Wo + wo) * g.Kpad + (r * g.KW + s2) * g.C + c8 * 8, f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += f[j];
        }
      }
      st8(dx + static_cast<long long>(pix) * g.C + c8 * 8, acc);
    }
  }
}

// y[n, ho, wo, :] = x[n, ho*s, wo*s, :]   (scatter = 1: the transpose, dx zero elsewhere)
__global__ void __launch_bounds__(256)
subsample_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int N, int H, int W, int C,
                 int stride, int scatter) {
  const int cvec = C / 8;
  const int Ho = (H + stride - 1) / stride, Wo = (W + stride - 1) / stride;
  if (!scatter) {
    const long long total = static_cast<long long>(N) * Ho * Wo * cvec;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const int c8 = static_cast<int>(i % cvec);
      long long pix = i / cvec;
      const int wo = static_cast<int>(pix % Wo), ho = static_cast<int>((pix / Wo) % Ho);
      const long long n = pix / (static_cast<long long>(Wo) * Ho);
      *reinterpret_cast<uint4*>(out + pix * C + c8 * 8) =
          *reinterpret_cast<const uint4*>(in + ((n * H + ho * stride) * W + wo * stride) * C + c8 * 8);
    }
  } else {
    const long long total = static_cast<long long>(N) * H * W * cvec;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const int c8 = static_cast<int>(i % cvec);
      long long pix = i / cvec;
      const int w = static_cast<int>(pix % W), h = static_cast<int>((pix / W) % H);
      const long long n = pix / (static_cast<long long>(W) * H);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h % stride == 0 && w % stride == 0)
        v = *reinterpret_cast<const uint4*>(in + ((n * Ho + h / stride) * Wo + w / stride) * C + c8 * 8);
      *reinterpret_cast<uint4*>(out + pix * C + c8 * 8) = v;
    }
  }
}

// ------------------------------------ BatchNorm ---------------------------------------------
// Layout of the partial-sum kernels: eight threads cover 128 contiguous bytes of a row (eight channels each), the
// 32 thread groups of a block take every 32nd row of the slice, and the 32 partial sums of a channel meet in shared
// memory at the end.
__device__ __forceinline__ void bn_fold_and_store(float (&acc1)[8], float (&acc2)[8], float* __restrict__ part, int C,
                                                  int c_block0) {
  __shared__ float red[2][32][64];
  const int lane8 = threadIdx.x & 7, rowlane = threadIdx.x >> 3;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    red[0][rowlane][lane8 * 8 + j] = acc1[j];
    red[1][rowlane][lane8 * 8 + j] = acc2[j];
  }
  __syncthreads();
  if (threadIdx.x < 128) {
    const int which = threadIdx.x >> 6, ch = threadIdx.x & 63;
    float t = 0.f;
#pragma unroll 8
    for (int k = 0; k < 32; ++k) t += red[which][k][ch];
    if (c_block0 + ch < C) part[(static_cast<long long>(blockIdx.y) * 2 + which) * C + c_block0 + ch] = t;
  }
}

// part[slice][0][c] = sum x, part[slice][1][c] = sum x^2 over the slice's rows; x is [rows, C].
__global__ void __launch_bounds__(256)
bn_stats_partial_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ part, long long rows, int C,
                        int rows_per_slice) {
  const int c0 = (blockIdx.x * 8 + (threadIdx.x & 7)) * 8;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_slice;
  const long long r1 = min(rows, r0 + rows_per_slice);
  float a[8], b[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = b[j] = 0.f;
  if (c0 < C) {
    long long r = r0 + (threadIdx.x >> 3);
    for (; r + 96 < r1; r += 128) {                 // four independent rows in flight per thread
      float v[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) ld8(x + (r + 32 * u) * C + c0, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) { a[j] += v[u][j]; b[j] += v[u][j] * v[u][j]; }
    }
    for (; r < r1; r += 32) {
      float v[8];
      ld8(x + r * C + c0, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) { a[j] += v[j]; b[j] += v[j] * v[j]; }
    }
  }
  bn_fold_and_store(a, b, part, C, blockIdx.x * 64);
}

// mean / rstd per channel from the partials; also updates the running statistics.  Block = 32 channels x 8 groups
// of slices (a thread adds every eighth slice in double precision; the eight sums meet in shared memory).
__global__ void __launch_bounds__(256)
bn_stats_final_kernel(const float* __restrict__ part, int slices, int C, long long rows, float eps, float momentum,
                      float* __restrict__ mean, float* __restrict__ rstd, float* __restrict__ run_mean,
                      float* __restrict__ run_var) {
  __shared__ double ss[8][32], qq[8][32];
  const int cl = threadIdx.x & 31, sg = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cl;
  double s = 0.0, q = 0.0;
  if (c < C)
    for (int k = sg; k < slices; k += 8) {
      s += part[static_cast<long long>(k) * 2 * C + c];
      q += part[static_cast<long long>(k) * 2 * C + C + c];
    }
  ss[sg][cl] = s;
  qq[sg][cl] = q;
  __syncthreads();
  if (sg != 0 || c >= C) return;
  s = 0.0;
  q = 0.0;
#pragma unroll
  for (int k = 0; k < 8; ++k) { s += ss[k][cl]; q += qq[k][cl]; }
  const double m = s / static_cast<double>(rows);
  double var = q / static_cast<double>(rows) - m * m;
  if (var < 0.0) var = 0.0;
  mean[c] = static_cast<float>(m);
  rstd[c] = rsqrtf(static_cast<float>(var) + eps);
  if (run_mean != nullptr) {
    const double unbiased = rows > 1 ? var * static_cast<double>(rows) / static_cast<double>(rows - 1) : var;
    run_mean[c] = (1.f - momentum) * run_mean[c] + momentum * static_cast<float>(m);
    run_var[c] = (1.f - momentum) * run_var[c] + momentum * static_cast<float>(unbiased);
  }
}

// Thread layout of the two element-wise BatchNorm passes: eight consecutive threads cover 128 contiguous bytes of a
// row (eight channels each), a block of 256 threads covers 32 rows of one 64-channel column block and walks down
// the rows.  A thread's channels never change, so the per-channel constants are loaded once into registers; an
// earlier form that recomputed the channel from a flat index read them again for every 16 bytes of data, and those
// reads (a kilobyte per warp and array) kept the L1 busy while DRAM ran at 11 % of its peak.
constexpr int kBnRowsPerBlock = 32;
inline dim3 bn_grid(long long rows, int C, int num_sms) {
  const int gx = (C / 8 + 7) / 8;
  long long gy = (rows + kBnRowsPerBlock - 1) / kBnRowsPerBlock;
  const long long cap = (static_cast<long long>(num_sms) * 16 + gx - 1) / gx;
  if (gy > cap) gy = cap;
  if (gy < 1) gy = 1;
  if (gy > 65535) gy = 65535;
  return dim3(gx, static_cast<unsigned>(gy));
}

// y = [relu]((x - mean) * rstd * gamma + beta [+ residual])
__global__ void __launch_bounds__(256)
bn_apply_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                const float* __restrict__ mean, const float* __restrict__ rstd, const float* __restrict__ gamma,
                const float* __restrict__ beta, __nv_bfloat16* __restrict__ y, long long rows, int C, int relu) {
  const int cv = blockIdx.x * 8 + (threadIdx.x & 7);
  if (cv >= C / 8) return;
  const int c0 = cv * 8;
  float a[8], b[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    a[j] = rstd[c0 + j] * gamma[c0 + j];
    b[j] = beta[c0 + j] - mean[c0 + j] * a[j];
  }
  const long long stride = static_cast<long long>(gridDim.y) * kBnRowsPerBlock;
  long long r = static_cast<long long>(blockIdx.y) * kBnRowsPerBlock + (threadIdx.x >> 3);
  auto finish = [&](long long row, float (&f)[8], const float (&res)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      f[j] = f[j] * a[j] + b[j] + res[j];
      if (relu) f[j] = fmaxf(f[j], 0.f);
    }
    st8(y + row * C + c0, f);
  };
  for (; r + 3 * stride < rows; r += 4 * stride) {   // four independent rows in flight per thread
    float f[4][8], q[4][8];
#pragma unroll
    for (int u = 0; u < 4; ++u) ld8(x + (r + u * stride) * C + c0, f[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (residual != nullptr) {
        ld8(residual + (r + u * stride) * C + c0, q[u]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) q[u][j] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) finish(r + u * stride, f[u], q[u]);
  }
  for (; r < rows; r += stride) {
    float f[8], q[8];
    ld8(x + r * C + c0, f);
    if (residual != nullptr) {
      ld8(residual + r * C + c0, q);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = 0.f;
    }
    finish(r, f, q);
  }
}

// Backward partials over a row slice: sum g and sum g * xhat, with g = dy masked by (y > 0) when relu.
__global__ void __launch_bounds__(256)
bn_bwd_partial_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const __nv_bfloat16* __restrict__ y, const float* __restrict__ mean,
                      const float* __restrict__ rstd, float* __restrict__ part, long long rows, int C,
                      int rows_per_slice, int relu) {
  const int c0 = (blockIdx.x * 8 + (threadIdx.x & 7)) * 8;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_slice;
  const long long r1 = min(rows, r0 + rows_per_slice);
  float a[8], b[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = b[j] = 0.f;
  if (c0 < C) {
    float m[8], q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { m[j] = mean[c0 + j]; q[j] = rstd[c0 + j]; }
    auto add = [&](float (&g)[8], const float (&v)[8], const float (&o)[8]) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (relu && !(o[j] > 0.f)) g[j] = 0.f;
        a[j] += g[j];
        b[j] += g[j] * (v[j] - m[j]) * q[j];
      }
    };
    long long r = r0 + (threadIdx.x >> 3);
    for (; r + 32 < r1; r += 64) {                  // two independent rows (up to six loads) in flight per thread
      float g[2][8], v[2][8], o[2][8];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        ld8(dy + (r + 32 * u) * C + c0, g[u]);
        ld8(x + (r + 32 * u) * C + c0, v[u]);
        if (relu) {
          ld8(y + (r + 32 * u) * C + c0, o[u]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[u][j] = 1.f;
        }
      }
      add(g[0], v[0], o[0]);
      add(g[1], v[1], o[1]);
    }
    for (; r < r1; r += 32) {
      float g[8], v[8], o[8];
      ld8(dy + r * C + c0, g);
      ld8(x + r * C + c0, v);
      if (relu) {
        ld8(y + r * C + c0, o);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = 1.f;
      }
      add(g, v, o);
    }
  }
  bn_fold_and_store(a, b, part, C, blockIdx.x * 64);
}

// sums[0][c] = sum g, sums[1][c] = sum g*xhat; dgamma (+)= sums[1], dbeta (+)= sums[0].  Same block layout as the
// forward's final kernel; the eight group sums are added in a fixed order.
__global__ void __launch_bounds__(256)
bn_bwd_final_kernel(const float* __restrict__ part, int slices, int C, float* __restrict__ sums,
                    float* __restrict__ dgamma, float* __restrict__ dbeta, int accumulate) {
  __shared__ float ss[8][32], qq[8][32];
  const int cl = threadIdx.x & 31, sg = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cl;
  float s = 0.f, q = 0.f;
  if (c < C)
    for (int k = sg; k < slices; k += 8) {
      s += part[static_cast<long long>(k) * 2 * C + c];
      q += part[static_cast<long long>(k) * 2 * C + C + c];
    }
  ss[sg][cl] = s;
  qq[sg][cl] = q;
  __syncthreads();
  if (sg != 0 || c >= C) return;
  s = 0.f;
  q = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) { s += ss[k][cl]; q += qq[k][cl]; }
  sums[c] = s;
  sums[C + c] = q;
  dbeta[c] = accumulate ? dbeta[c] + s : s;
  dgamma[c] = accumulate ? dgamma[c] + q : q;
}

// dx = gamma * rstd * (g - mean(g) - xhat * mean(g * xhat)); dres = g (when a residual was added).
// Per channel this is dx = A g + B x + D with A = gamma rstd, B = -A rstd mean(g xhat), D = -A mean(g) - B mean.
__global__ void __launch_bounds__(256)
bn_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                 const __nv_bfloat16* __restrict__ y, const float* __restrict__ mean, const float* __restrict__ rstd,
                 const float* __restrict__ gamma, const float* __restrict__ sums, __nv_bfloat16* __restrict__ dx,
                 __nv_bfloat16* __restrict__ dres, long long rows, int C, int relu) {
  const int cv = blockIdx.x * 8 + (threadIdx.x & 7);
  if (cv >= C / 8) return;
  const int c0 = cv * 8;
  const float inv_n = 1.0f / static_cast<float>(rows);
  float A[8], Bc[8], D[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = c0 + j;
    A[j] = gamma[c] * rstd[c];
    Bc[j] = -A[j] * rstd[c] * sums[C + c] * inv_n;
    D[j] = -A[j] * sums[c] * inv_n - Bc[j] * mean[c];
  }
  const long long stride = static_cast<long long>(gridDim.y) * kBnRowsPerBlock;
  long long r = static_cast<long long>(blockIdx.y) * kBnRowsPerBlock + (threadIdx.x >> 3);
  auto finish = [&](long long row, float (&g)[8], const float (&v)[8], const float (&yy)[8]) {
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (relu && !(yy[j] > 0.f)) g[j] = 0.f;
      o[j] = A[j] * g[j] + Bc[j] * v[j] + D[j];
    }
    st8(dx + row * C + c0, o);
    if (dres != nullptr) st8(dres + row * C + c0, g);
  };
  for (; r + stride < rows; r += 2 * stride) {       // two independent rows (up to six loads) in flight per thread
    float g[2][8], v[2][8], yy[2][8];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      ld8(dy + (r + u * stride) * C + c0, g[u]);
      ld8(x + (r + u * stride) * C + c0, v[u]);
      if (relu) {
        ld8(y + (r + u * stride) * C + c0, yy[u]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) yy[u][j] = 1.f;
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) finish(r + u * stride, g[u], v[u], yy[u]);
  }
  for (; r < rows; r += stride) {
    float g[8], v[8], yy[8];
    ld8(dy + r * C + c0, g);
    ld8(x + r * C + c0, v);
    if (relu) {
      ld8(y + r * C + c0, yy);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) yy[j] = 1.f;
    }
    finish(r, g, v, yy);
  }
}

// ------------------------------------- pooling ----------------------------------------------
// 3x3 / stride 2 / pad 1 max pooling; idx stores the winning tap (0..8) for the backward pass.
__global__ void __launch_bounds__(256)
maxpool_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ idx,
                   int N, int H, int W, int C) {
  // eight channels per thread: 16-byte loads of up to nine taps, one 16-byte store of y and one 8-byte store of idx
  const int Ho = (H + 1) / 2, Wo = (W + 1) / 2, cvec = C / 8;
  const long long total = static_cast<long long>(N) * Ho * Wo * cvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c0 = static_cast<int>(i % cvec) * 8;
    const long long pix = i / cvec;
    const int wo = static_cast<int>(pix % Wo), ho = static_cast<int>((pix / Wo) % Ho);
    const long long n = pix / (static_cast<long long>(Wo) * Ho);
    float best[8];
    uint32_t arg[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; arg[j] = 4; }
#pragma unroll
    for (int r = 0; r < 3; ++r)
#pragma unroll
      for (int t = 0; t < 3; ++t) {
        const int h = ho * 2 + r - 1, w = wo * 2 + t - 1;
        if (h < 0 || h >= H || w < 0 || w >= W) continue;
        float v[8];
        ld8(x + ((n * H + h) * W + w) * C + c0, v);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (v[j] > best[j]) { best[j] = v[j]; arg[j] = r * 3 + t; }
      }
    st8(y + pix * C + c0, best);
    uint2 packed;
    packed.x = arg[0] | (arg[1] << 8) | (arg[2] << 16) | (arg[3] << 24);
    packed.y = arg[4] | (arg[5] << 8) | (arg[6] << 16) | (arg[7] << 24);
    *reinterpret_cast<uint2*>(idx + pix * C + c0) = packed;
  }
}

__global__ void __launch_bounds__(256)
maxpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const uint8_t* __restrict__ idx,
                   __nv_bfloat16* __restrict__ dx, int N, int H, int W, int C) {
  const int Ho = (H + 1) / 2, Wo = (W + 1) / 2, cvec = C / 8;
  const long long total = static_cast<long long>(N) * H * W * cvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c0 = static_cast<int>(i % cvec) * 8;
    const long long pix = i / cvec;
    const int w = static_cast<int>(pix % W), h = static_cast<int>((pix / W) % H);
    const long long n = pix / (static_cast<long long>(W) * H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // output windows (ho, wo) that contain (h, w): ho*2 - 1 <= h <= ho*2 + 1
    for (int ho = h / 2; ho <= (h + 1) / 2; ++ho) {
      if (ho >= Ho) continue;
      const uint32_t r = h - ho * 2 + 1;
      for (int wo = w / 2; wo <= (w + 1) / 2; ++wo) {
        if (wo >= Wo) continue;
        const uint32_t tap = r * 3 + (w - wo * 2 + 1);
        const long long o = ((n * Ho + ho) * Wo + wo) * C + c0;
        const uint2 packed = *reinterpret_cast<const uint2*>(idx + o);
        float g[8];
        ld8(dy + o, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t a = ((j < 4 ? packed.x : packed.y) >> (8 * (j & 3))) & 0xFFu;
          if (a == tap) acc[j] += g[j];
        }
      }
    }
    st8(dx + pix * C + c0, acc);
  }
}

// y[n, c] = mean over hw of x[n, hw, c]; backward broadcasts dy / HW.
__global__ void __launch_bounds__(256)
avgpool_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int N, int HW, int C) {
  const long long total = static_cast<long long>(N) * C;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % C);
    const long long n = i / C;
    float s = 0.f;
    for (int p = 0; p < HW; ++p) s += __bfloat162float(x[(n * HW + p) * C + c]);
    y[i] = __float2bfloat16(s / static_cast<float>(HW));
  }
}
__global__ void __launch_bounds__(256)
avgpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, int N, int HW, int C) {
  const long long total = static_cast<long long>(N) * HW * C;
  const float inv = 1.0f / static_cast<float>(HW);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % C);
    const long long n = i / (static_cast<long long>(HW) * C);
    dx[i] = __float2bfloat16(__bfloat162float(dy[n * C + c]) * inv);
  }
}

int grid_for(long long work, int num_sms) {
  long long want = (work + 255) / 256;
  return static_cast<int>(want < 1 ? 1 : (want > num_sms * 32LL ? num_sms * 32LL : want));
}

}  // namespace

int bn_slices(long long rows) {
  long long s = (rows + 511) / 512;
  return static_cast<int>(s < 1 ? 1 : (s > 256 ? 256 : s));
}

int im2col_launch(const void* x, void* cols, int N, int H, int W, int C, int KH, int KW, int stride, int pad, int Kpad,
                  int num_sms, cudaStream_t stream) {
  ConvGeom g{N, H, W, C, KH, KW, stride, pad, (H + 2 * pad - KH) / stride + 1, (W + 2 * pad - KW) / stride + 1, Kpad};
  const auto* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto* cb = reinterpret_cast<__nv_bfloat16*>(cols);
  if (C % 8 == 0 && Kpad == KH * KW * C) {
    const long long rows = static_cast<long long>(N) * g.Ho * g.Wo;
    if (rows > 0x7fffffffLL) return -3;
    const int blocks = static_cast<int>(rows < num_sms * 16LL ? rows : num_sms * 16LL);
    im2col_kernel<<<blocks, 256, 0, stream>>>(xb, cb, g);
  } else {
    const long long work = static_cast<long long>(N) * g.Ho * g.Wo * Kpad;
    im2col_small_c_kernel<<<grid_for(work, num_sms), 256, 0, stream>>>(xb, cb, g);
  }
  return static_cast<int>(cudaGetLastError());
}

int col2im_launch(const void* dcols, void* dx, int N, int H, int W, int C, int KH, int KW, int stride, int pad, int Kpad,
                  int num_sms, cudaStream_t stream) {
  if (C % 8) return -3;
  ConvGeom g{N, H, W, C, KH, KW, stride, pad, (H + 2 * pad - KH) / stride + 1, (W + 2 * pad - KW) / stride + 1, Kpad};
  const long long pixels = static_cast<long long>(N) * H * W;
  if (pixels > 0x7fffffffLL) return -3;
  const int cvec = C / 8, ppb = cvec >= 256 ? 1 : 256 / cvec;
  const long long want = (pixels + ppb - 1) / ppb;
  col2im_kernel<<<static_cast<int>(want < num_sms * 16LL ? want : num_sms * 16LL), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dcols),
                                                             reinterpret_cast<__nv_bfloat16*>(dx), g);
  return static_cast<int>(cudaGetLastError());
}

int subsample_launch(const void* in, void* out, int N, int H, int W, int C, int stride, int scatter, int num_sms,
                     cudaStream_t stream) {
  if (C % 8) return -3;
  const long long work = static_cast<long long>(N) * H * W * (C / 8);
  subsample_kernel<<<grid_for(work, num_sms), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(in),
                                                                reinterpret_cast<__nv_bfloat16*>(out), N, H, W, C,
                                                                stride, scatter);
  return static_cast<int>(cudaGetLastError());
}

// part: scratch of bn_slices(rows) * 2 * C floats.
int bn_fwd_launch(const void* x, const void* residual, const float* gamma, const float* beta, void* y, float* mean,
                  float* rstd, float* run_mean, float* run_var, float* part, long long rows, int C, float eps,
                  float momentum, int relu, int num_sms, cudaStream_t stream) {
  if (C % 8) return -3;
  const int slices = bn_slices(rows);
  const int rps = static_cast<int>((rows + slices - 1) / slices);
  dim3 grid((C / 8 + 7) / 8, slices);
  bn_stats_partial_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), part, rows, C, rps);
  bn_stats_final_kernel<<<(C + 31) / 32, 256, 0, stream>>>(part, slices, C, rows, eps, momentum, mean, rstd,
                                                             run_mean, run_var);
  bn_apply_kernel<<<bn_grid(rows, C, num_sms), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(residual), mean, rstd, gamma,
      beta, reinterpret_cast<__nv_bfloat16*>(y), rows, C, relu);
  return static_cast<int>(cudaGetLastError());
}

// y = [relu](gamma * (x - mean) * rstd + beta [+ residual]) with GIVEN per-channel statistics (inference: the running
// estimates); no statistics pass, nothing updated.
int bn_apply_launch(const void* x, const void* residual, const float* mean, const float* rstd, const float* gamma,
                    const float* beta, void* y, long long rows, int C, int relu, int num_sms, cudaStream_t stream) {
  if (C % 8) return -3;
  bn_apply_kernel<<<bn_grid(rows, C, num_sms), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(residual), mean, rstd, gamma,
      beta, reinterpret_cast<__nv_bfloat16*>(y), rows, C, relu);
  return static_cast<int>(cudaGetLastError());
}

// sums: scratch of 2 * C floats; part as above.
int bn_bwd_launch(const void* dy, const void* x, const void* y, const float* mean, const float* rstd,
                  const float* gamma, void* dx, void* dres, float* dgamma, float* dbeta, float* part, float* sums,
                  int accumulate, long long rows, int C, int relu, int num_sms, cudaStream_t stream) {
  if (C % 8) return -3;
  const int slices = bn_slices(rows);
  const int rps = static_cast<int>((rows + slices - 1) / slices);
  dim3 grid((C / 8 + 7) / 8, slices);
  bn_bwd_partial_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dy),
                                                  reinterpret_cast<const __nv_bfloat16*>(x),
                                                  reinterpret_cast<const __nv_bfloat16*>(y), mean, rstd, part, rows,
                                                  C, rps, relu);
  bn_bwd_final_kernel<<<(C + 31) / 32, 256, 0, stream>>>(part, slices, C, sums, dgamma, dbeta, accumulate);
  bn_bwd_dx_kernel<<<bn_grid(rows, C, num_sms), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x),
      reinterpret_cast<const __nv_bfloat16*>(y), mean, rstd, gamma, sums, reinterpret_cast<__nv_bfloat16*>(dx),
      reinterpret_cast<__nv_bfloat16*>(dres), rows, C, relu);
  return static_cast<int>(cudaGetLastError());
}

int maxpool_fwd_launch(const void* x, void* y, void* idx, int N, int H, int W, int C, int num_sms, cudaStream_t stream) {
  if (C % 8) return -3;
  const long long work = static_cast<long long>(N) * ((H + 1) / 2) * ((W + 1) / 2) * (C / 8);
  maxpool_fwd_kernel<<<grid_for(work, num_sms), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                                  reinterpret_cast<__nv_bfloat16*>(y),
                                                                  reinterpret_cast<uint8_t*>(idx), N, H, W, C);
  return static_cast<int>(cudaGetLastError());
}
int maxpool_bwd_launch(const void* dy, const void* idx, void* dx, int N, int H, int W, int C, int num_sms,
                       cudaStream_t stream) {
  if (C % 8) return -3;
  const long long work = static_cast<long long>(N) * H * W * (C / 8);
  maxpool_bwd_kernel<<<grid_for(work, num_sms), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dy),
                                                                  reinterpret_cast<const uint8_t*>(idx),
                                                                  reinterpret_cast<__nv_bfloat16*>(dx), N, H, W, C);
  return static_cast<int>(cudaGetLastError());
}
int avgpool_launch(const void* in, void* out, int N, int HW, int C, int backward, int num_sms, cudaStream_t stream) {
  if (!backward)
    avgpool_fwd_kernel<<<grid_for(static_cast<long long>(N) * C, num_sms), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), N, HW, C);
  else
    avgpool_bwd_kernel<<<grid_for(static_cast<long long>(N) * HW * C, num_sms), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), N, HW, C);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ssb
