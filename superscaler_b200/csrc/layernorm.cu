// LayerNorm forward / backward for bf16 activations with fp32 statistics, one warp per row.
// Covers the role of the reference's mixed-precision fused LayerNorm extension
// (runtime/megatron/fused_kernels/layer_norm_cuda_kernel.cu:290-334 forward,
// :415-651 backward): y = (x - mean) * rstd * gamma + beta, saving mean and rstd;
// backward produces dx and per-column partial sums for dgamma / dbeta that a
// second small kernel folds (deterministic, no atomics).
//
// HBM-bound: every kernel moves 16 bytes per lane per access and keeps the row in
// registers between the statistics pass and the normalisation pass.
#include "common.cuh"

namespace ssb {

constexpr int kColsumTickets = 4096;   // column blocks of 256 that one column-sum call may cover in one pass
int colsum_tickets() { return kColsumTickets; }
namespace {

constexpr int kLnWarpsPerBlock = 4;

// VPL = uint4 vectors (8 bf16) per lane; H = VPL * 256.  VPL == 0 selects the generic
// path that re-reads the row (any H that is a multiple of 8).
template <int VPL>
__global__ void __launch_bounds__(kLnWarpsPerBlock * 32)
ln_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
              const float* __restrict__ gamma, const float* __restrict__ beta, __nv_bfloat16* __restrict__ y,
              __nv_bfloat16* __restrict__ sum_out, float* __restrict__ mean_out, float* __restrict__ rstd_out,
              int rows, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * kLnWarpsPerBlock + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * kLnWarpsPerBlock;
  const int nvec = H / 8;
  for (int row = warp_global; row < rows; row += warps_total) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + static_cast<size_t>(row) * H) : nullptr;
    uint4* sr = sum_out ? reinterpret_cast<uint4*>(sum_out + static_cast<size_t>(row) * H) : nullptr;
    constexpr int NV = VPL > 0 ? VPL : 1;
    float vals[NV][8];
    float s = 0.f;
    if (VPL > 0) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        uint4 q = xr[i * 32 + lane];
        float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
        vals[i][0] = f0.x; vals[i][1] = f0.y; vals[i][2] = f1.x; vals[i][3] = f1.y;
        vals[i][4] = f2.x; vals[i][5] = f2.y; vals[i][6] = f3.x; vals[i][7] = f3.y;
        if (rr) {
          uint4 r = rr[i * 32 + lane];
          float2 g0 = unpack_bf16x2(r.x), g1 = unpack_bf16x2(r.y), g2 = unpack_bf16x2(r.z), g3 = unpack_bf16x2(r.w);
          vals[i][0] += g0.x; vals[i][1] += g0.y; vals[i][2] += g1.x; vals[i][3] += g1.y;
          vals[i][4] += g2.x; vals[i][5] += g2.y; vals[i][6] += g3.x; vals[i][7] += g3.y;
          uint4 o;
          o.x = pack_bf16x2(vals[i][0], vals[i][1]); o.y = pack_bf16x2(vals[i][2], vals[i][3]);
          o.z = pack_bf16x2(vals[i][4], vals[i][5]); o.w = pack_bf16x2(vals[i][6], vals[i][7]);
          if (sr) sr[i * 32 + lane] = o;
          // statistics are taken on the rounded sum so that forward and backward see the same x
          float2 h0 = unpack_bf16x2(o.x), h1 = unpack_bf16x2(o.y), h2 = unpack_bf16x2(o.z), h3 = unpack_bf16x2(o.w);
          vals[i][0] = h0.x; vals[i][1] = h0.y; vals[i][2] = h1.x; vals[i][3] = h1.y;
          vals[i][4] = h2.x; vals[i][5] = h2.y; vals[i][6] = h3.x; vals[i][7] = h3.y;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) s += vals[i][j];
      }
    } else {
      for (int v = lane; v < nvec; v += 32) {
        uint4 q = xr[v];
        float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
        float e[8] = {f0.x, f0.y, f1.x, f1.y, f2.x, f2.y, f3.x, f3.y};
        if (rr) {
          uint4 r = rr[v];
          float2 g0 = unpack_bf16x2(r.x), g1 = unpack_bf16x2(r.y), g2 = unpack_bf16x2(r.z), g3 = unpack_bf16x2(r.w);
          e[0] += g0.x; e[1] += g0.y; e[2] += g1.x; e[3] += g1.y; e[4] += g2.x; e[5] += g2.y; e[6] += g3.x; e[7] += g3.y;
          uint4 o;
          o.x = pack_bf16x2(e[0], e[1]); o.y = pack_bf16x2(e[2], e[3]);
          o.z = pack_bf16x2(e[4], e[5]); o.w = pack_bf16x2(e[6], e[7]);
          if (sr) sr[v] = o;
          float2 h0 = unpack_bf16x2(o.x), h1 = unpack_bf16x2(o.y), h2 = unpack_bf16x2(o.z), h3 = unpack_bf16x2(o.w);
          e[0] = h0.x; e[1] = h0.y; e[2] = h1.x; e[3] = h1.y; e[4] = h2.x; e[5] = h2.y; e[6] = h3.x; e[7] = h3.y;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) s += e[j];
      }
    }
    const float mean = warp_sum(s) / static_cast<float>(H);
    float sq = 0.f;
    // The generic path reads the (possibly just written) sum back; make the stores visible to the warp.
    const uint4* src = (VPL == 0 && rr && sr) ? reinterpret_cast<const uint4*>(sr) : xr;
    if (VPL == 0 && rr && sr) __syncwarp();
    if (VPL > 0) {
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = vals[i][j] - mean;
          sq += d * d;
        }
    } else {
      for (int v = lane; v < nvec; v += 32) {
        uint4 q = src[v];
        float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
        float e[8] = {f0.x, f0.y, f1.x, f1.y, f2.x, f2.y, f3.x, f3.y};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = e[j] - mean;
          sq += d * d;
        }
      }
    }
    const float var = warp_sum(sq) / static_cast<float>(H);
    const float rstd = rsqrtf(var + eps);
    if (lane == 0) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
    uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H);
    if (VPL > 0) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int v = i * 32 + lane;
        const float4 g0 = reinterpret_cast<const float4*>(gamma)[2 * v], g1 = reinterpret_cast<const float4*>(gamma)[2 * v + 1];
        const float4 b0 = reinterpret_cast<const float4*>(beta)[2 * v], b1 = reinterpret_cast<const float4*>(beta)[2 * v + 1];
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (vals[i][j] - mean) * rstd * g[j] + b[j];
        uint4 q;
        q.x = pack_bf16x2(o[0], o[1]); q.y = pack_bf16x2(o[2], o[3]);
        q.z = pack_bf16x2(o[4], o[5]); q.w = pack_bf16x2(o[6], o[7]);
        yr[v] = q;
      }
    } else {
      for (int v = lane; v < nvec; v += 32) {
        uint4 q = src[v];
        float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
        float e[8] = {f0.x, f0.y, f1.x, f1.y, f2.x, f2.y, f3.x, f3.y};
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (e[j] - mean) * rstd * gamma[v * 8 + j] + beta[v * 8 + j];
        uint4 w;
        w.x = pack_bf16x2(o[0], o[1]); w.y = pack_bf16x2(o[2], o[3]);
        w.z = pack_bf16x2(o[4], o[5]); w.w = pack_bf16x2(o[6], o[7]);
        yr[v] = w;
      }
    }
  }
}

// dx = rstd * (dy*gamma - mean_H(dy*gamma) - xhat * mean_H(dy*gamma*xhat)) (+ dresidual)
__global__ void __launch_bounds__(kLnWarpsPerBlock * 32)
ln_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                 const float* __restrict__ gamma, const float* __restrict__ mean, const float* __restrict__ rstd,
                 const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, int rows, int H) {
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * kLnWarpsPerBlock + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * kLnWarpsPerBlock;
  const int nvec = H / 8;
  for (int row = warp_global; row < rows; row += warps_total) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * H);
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 qd = dyr[v], qx = xr[v];
      const float2 d0 = unpack_bf16x2(qd.x), d1 = unpack_bf16x2(qd.y), d2 = unpack_bf16x2(qd.z), d3 = unpack_bf16x2(qd.w);
      const float2 x0 = unpack_bf16x2(qx.x), x1 = unpack_bf16x2(qx.y), x2 = unpack_bf16x2(qx.z), x3 = unpack_bf16x2(qx.w);
      const float d[8] = {d0.x, d0.y, d1.x, d1.y, d2.x, d2.y, d3.x, d3.y};
      const float xv[8] = {x0.x, x0.y, x1.x, x1.y, x2.x, x2.y, x3.x, x3.y};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float dg = d[j] * gamma[v * 8 + j];
        s1 += dg;
        s2 += dg * (xv[j] - mu) * rs;
      }
    }
    s1 = warp_sum(s1) / static_cast<float>(H);
    s2 = warp_sum(s2) / static_cast<float>(H);
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * H);
    const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + static_cast<size_t>(row) * H) : nullptr;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 qd = dyr[v], qx = xr[v];
      const float2 d0 = unpack_bf16x2(qd.x), d1 = unpack_bf16x2(qd.y), d2 = unpack_bf16x2(qd.z), d3 = unpack_bf16x2(qd.w);
      const float2 x0 = unpack_bf16x2(qx.x), x1 = unpack_bf16x2(qx.y), x2 = unpack_bf16x2(qx.z), x3 = unpack_bf16x2(qx.w);
      const float d[8] = {d0.x, d0.y, d1.x, d1.y, d2.x, d2.y, d3.x, d3.y};
      const float xv[8] = {x0.x, x0.y, x1.x, x1.y, x2.x, x2.y, x3.x, x3.y};
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xhat = (xv[j] - mu) * rs;
        o[j] = rs * (d[j] * gamma[v * 8 + j] - s1 - xhat * s2);
      }
      if (drr) {
        const uint4 qr = drr[v];
        const float2 r0 = unpack_bf16x2(qr.x), r1 = unpack_bf16x2(qr.y), r2 = unpack_bf16x2(qr.z), r3 = unpack_bf16x2(qr.w);
        o[0] += r0.x; o[1] += r0.y; o[2] += r1.x; o[3] += r1.y; o[4] += r2.x; o[5] += r2.y; o[6] += r3.x; o[7] += r3.y;
      }
      uint4 w;
      w.x = pack_bf16x2(o[0], o[1]); w.y = pack_bf16x2(o[2], o[3]);
      w.z = pack_bf16x2(o[4], o[5]); w.w = pack_bf16x2(o[6], o[7]);
      dxr[v] = w;
    }
  }
}

// One pass over dy and x for H = VPL * 256 * WPR: dx, and in the same sweep every lane keeps running sums of
// dy * xhat and dy for its 8 * VPL columns over all rows its warp visits.  WPR warps share a row (each owns a
// contiguous part of the columns, so that the running sums fit in registers) and exchange their two row sums through
// shared memory.  The warps of a block fold their column sums through shared memory in a fixed order and the block
// writes ONE row of partials (part_g[block][h], part_b[block][h]); fold_partials_kernel adds the blocks.  dy and x
// are read once instead of twice, and the result does not depend on the order of execution.
template <int VPL, int WPR>
__global__ void __launch_bounds__(kLnWarpsPerBlock * 32)
ln_bwd_onepass_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const float* __restrict__ gamma, const float* __restrict__ mean, const float* __restrict__ rstd,
                      const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                      float* __restrict__ part_g, float* __restrict__ part_b, int rows, int H) {
  constexpr int RPB = kLnWarpsPerBlock / WPR;        // rows a block works on at a time
  __shared__ float fold_g[VPL * 256 * WPR], fold_b[VPL * 256 * WPR];
  __shared__ float xch[2][RPB][WPR][2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rslot = warp / WPR, part = warp % WPR;
  const int v0 = part * VPL * 32;                    // first 16-byte vector of this warp's columns
  float ag[VPL][8], ab[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) ag[i][j] = ab[i][j] = 0.f;
  int it = 0;
  // every warp of a row slot runs the same number of iterations: the named barrier below is reached by all of them
  for (int row = blockIdx.x * RPB + rslot; row < rows; row += gridDim.x * RPB, ++it) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * H);
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    const float mu = mean[row], rs = rstd[row];
    uint4 qd[VPL], qx[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      qd[i] = dyr[v0 + i * 32 + lane];
      qx[i] = xr[v0 + i * 32 + lane];
    }
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = v0 + i * 32 + lane;
      const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * v);
      const float4 g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * v + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      const float2 d0 = unpack_bf16x2(qd[i].x), d1 = unpack_bf16x2(qd[i].y), d2 = unpack_bf16x2(qd[i].z), d3 = unpack_bf16x2(qd[i].w);
      const float2 x0 = unpack_bf16x2(qx[i].x), x1 = unpack_bf16x2(qx[i].y), x2 = unpack_bf16x2(qx[i].z), x3 = unpack_bf16x2(qx[i].w);
      const float d[8] = {d0.x, d0.y, d1.x, d1.y, d2.x, d2.y, d3.x, d3.y};
      const float xv[8] = {x0.x, x0.y, x1.x, x1.y, x2.x, x2.y, x3.x, x3.y};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xhat = (xv[j] - mu) * rs;
        const float dg = d[j] * g[j];
        s1 += dg;
        s2 += dg * xhat;
        ag[i][j] += d[j] * xhat;
        ab[i][j] += d[j];
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if constexpr (WPR > 1) {
      float* slot = &xch[it & 1][rslot][0][0];
      if (lane == 0) {
        slot[part * 2] = s1;
        slot[part * 2 + 1] = s2;
      }
      asm volatile("bar.sync %0, %1;" ::"r"(1 + rslot), "r"(32 * WPR) : "memory");
      s1 = 0.f;
      s2 = 0.f;
#pragma unroll
      for (int w = 0; w < WPR; ++w) {
        s1 += slot[w * 2];
        s2 += slot[w * 2 + 1];
      }
    }
    s1 /= static_cast<float>(H);
    s2 /= static_cast<float>(H);
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * H);
    const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + static_cast<size_t>(row) * H) : nullptr;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = v0 + i * 32 + lane;
      const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * v);
      const float4 g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * v + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      const float2 d0 = unpack_bf16x2(qd[i].x), d1 = unpack_bf16x2(qd[i].y), d2 = unpack_bf16x2(qd[i].z), d3 = unpack_bf16x2(qd[i].w);
      const float2 x0 = unpack_bf16x2(qx[i].x), x1 = unpack_bf16x2(qx[i].y), x2 = unpack_bf16x2(qx[i].z), x3 = unpack_bf16x2(qx[i].w);
      const float d[8] = {d0.x, d0.y, d1.x, d1.y, d2.x, d2.y, d3.x, d3.y};
      const float xv[8] = {x0.x, x0.y, x1.x, x1.y, x2.x, x2.y, x3.x, x3.y};
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xhat = (xv[j] - mu) * rs;
        o[j] = rs * (d[j] * g[j] - s1 - xhat * s2);
      }
      if (drr) {
        const uint4 qr = drr[v];
        const float2 r0 = unpack_bf16x2(qr.x), r1 = unpack_bf16x2(qr.y), r2 = unpack_bf16x2(qr.z), r3 = unpack_bf16x2(qr.w);
        o[0] += r0.x; o[1] += r0.y; o[2] += r1.x; o[3] += r1.y; o[4] += r2.x; o[5] += r2.y; o[6] += r3.x; o[7] += r3.y;
      }
      uint4 w;
      w.x = pack_bf16x2(o[0], o[1]); w.y = pack_bf16x2(o[2], o[3]);
      w.z = pack_bf16x2(o[4], o[5]); w.w = pack_bf16x2(o[6], o[7]);
      dxr[v] = w;
    }
  }
  // fold the row slots of the block in the order 0, 1, ...: slot s adds its warps' sums to the columns they own
  for (int sl = 0; sl < RPB; ++sl) {
    if (rslot == sl) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int c = (v0 + i * 32 + lane) * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          fold_g[c + j] = (sl == 0 ? 0.f : fold_g[c + j]) + ag[i][j];
          fold_b[c + j] = (sl == 0 ? 0.f : fold_b[c + j]) + ab[i][j];
        }
      }
    }
    __syncthreads();
  }
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    part_g[static_cast<size_t>(blockIdx.x) * H + c] = fold_g[c];
    part_b[static_cast<size_t>(blockIdx.x) * H + c] = fold_b[c];
  }
}

// Partial column sums over a slice of rows: part_g[slice][h] = sum dy*xhat, part_b[slice][h] = sum dy.
// Block = 32 columns-pairs x 8 row lanes: thread (tx, ty) owns columns 2*(bx*32+tx), +1 and rows ty, ty+8, ...
__global__ void __launch_bounds__(256)
ln_bwd_gb_partial_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                         const float* __restrict__ mean, const float* __restrict__ rstd, float* __restrict__ part_g,
                         float* __restrict__ part_b, int rows, int H, int rows_per_slice) {
  __shared__ float sg[8][64], sb[8][64];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + tx) * 2;
  const int r0 = blockIdx.y * rows_per_slice;
  const int r1 = min(rows, r0 + rows_per_slice);
  float g0 = 0.f, g1 = 0.f, b0 = 0.f, b1 = 0.f;
  if (col < H) {
    for (int r = r0 + ty; r < r1; r += 8) {
      const uint32_t qd = *reinterpret_cast<const uint32_t*>(dy + static_cast<size_t>(r) * H + col);
      const uint32_t qx = *reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(r) * H + col);
      const float2 d = unpack_bf16x2(qd), xv = unpack_bf16x2(qx);
      const float mu = mean[r], rs = rstd[r];
      g0 += d.x * (xv.x - mu) * rs;
      g1 += d.y * (xv.y - mu) * rs;
      b0 += d.x;
      b1 += d.y;
    }
  }
  sg[ty][tx * 2] = g0; sg[ty][tx * 2 + 1] = g1;
  sb[ty][tx * 2] = b0; sb[ty][tx * 2 + 1] = b1;
  __syncthreads();
  if (ty == 0 && col < H) {
    float a0 = 0.f, a1 = 0.f, c0 = 0.f, c1 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      a0 += sg[k][tx * 2]; a1 += sg[k][tx * 2 + 1];
      c0 += sb[k][tx * 2]; c1 += sb[k][tx * 2 + 1];
    }
    part_g[static_cast<size_t>(blockIdx.y) * H + col] = a0;
    part_g[static_cast<size_t>(blockIdx.y) * H + col + 1] = a1;
    part_b[static_cast<size_t>(blockIdx.y) * H + col] = c0;
    part_b[static_cast<size_t>(blockIdx.y) * H + col + 1] = c1;
  }
}

// out[h] (+)= sum_slices part[slice][h]
__global__ void fold_partials_kernel(const float* __restrict__ part, float* __restrict__ out, int slices, int H,
                                     int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int k = 0; k < slices; ++k) s += part[static_cast<size_t>(k) * H + h];
  out[h] = accumulate ? out[h] + s : s;
}

// Both LayerNorm weight gradients in one launch: block (x, which) folds 64 columns of part_g (which = 0) or part_b
// (which = 1); its 256 threads are 64 columns x 4 groups of slices, added in a fixed order.
__global__ void __launch_bounds__(256)
fold_partials2_kernel(const float* __restrict__ part_g, const float* __restrict__ part_b, float* __restrict__ dgamma,
                      float* __restrict__ dbeta, int slices, int H, int accumulate) {
  __shared__ float sm[4][64];
  const float* part = blockIdx.y == 0 ? part_g : part_b;
  float* out = blockIdx.y == 0 ? dgamma : dbeta;
  const int c = threadIdx.x & 63, sg = threadIdx.x >> 6, h = blockIdx.x * 64 + c;
  float s = 0.f;
  if (h < H)
    for (int k = sg; k < slices; k += 4) s += part[static_cast<size_t>(k) * H + h];
  sm[sg][c] = s;
  __syncthreads();
  if (sg == 0 && h < H) {
    const float t = (sm[0][c] + sm[1][c]) + (sm[2][c] + sm[3][c]);
    out[h] = accumulate ? out[h] + t : t;
  }
}

// Column sum of a bf16 matrix [rows, N] (bias gradients) in ONE launch, for 16-byte aligned rows (N, lda multiples
// of 8).  A warp covers 512 contiguous bytes of a row (eight columns per lane), the eight warps of a block take
// every eighth row of the block's slice, and the block writes one row of partials for its 256 columns.  The block
// that finishes LAST for a column block (a ticket counter per column block, which it sets back to zero) adds the
// partials of all slices in slice order, so the result does not depend on which block that is.  The counters are
// shared by all calls on a device: calls must be ordered on one stream.
__global__ void __launch_bounds__(256)
colsum_onepass_kernel(const __nv_bfloat16* __restrict__ a, int lda, float* __restrict__ part, float* __restrict__ out,
                      int* __restrict__ tickets, int rows, int N, int rows_per_slice, int accumulate) {
  __shared__ float red[8][256 + 8];
  __shared__ int is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 256 + lane * 8;
  const int r0 = blockIdx.y * rows_per_slice;
  const int r1 = min(rows, r0 + rows_per_slice);
  float s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = 0.f;
  auto add = [&](const uint4& q) {
    const float2 v0 = unpack_bf16x2(q.x), v1 = unpack_bf16x2(q.y), v2 = unpack_bf16x2(q.z), v3 = unpack_bf16x2(q.w);
    s[0] += v0.x; s[1] += v0.y; s[2] += v1.x; s[3] += v1.y; s[4] += v2.x; s[5] += v2.y; s[6] += v3.x; s[7] += v3.y;
  };
  if (c0 < N) {
    int r = r0 + warp;
    for (; r + 24 < r1; r += 32) {                   // four independent rows in flight per thread
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) q[u] = *reinterpret_cast<const uint4*>(a + static_cast<size_t>(r + 8 * u) * lda + c0);
#pragma unroll
      for (int u = 0; u < 4; ++u) add(q[u]);
    }
    for (; r < r1; r += 8) add(*reinterpret_cast<const uint4*>(a + static_cast<size_t>(r) * lda + c0));
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = s[j];
  __syncthreads();
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col < N) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][threadIdx.x];
    part[static_cast<size_t>(blockIdx.y) * N + col] = t;
    __threadfence();
  }
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&tickets[blockIdx.x], 1) == static_cast<int>(gridDim.y) - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (col < N) {
    float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;      // four chains, joined in a fixed order
    const int n = static_cast<int>(gridDim.y);
    int k = 0;
    for (; k + 3 < n; k += 4) {
      t0 += __ldcg(part + static_cast<size_t>(k) * N + col);
      t1 += __ldcg(part + static_cast<size_t>(k + 1) * N + col);
      t2 += __ldcg(part + static_cast<size_t>(k + 2) * N + col);
      t3 += __ldcg(part + static_cast<size_t>(k + 3) * N + col);
    }
    for (; k < n; ++k) t0 += __ldcg(part + static_cast<size_t>(k) * N + col);
    const float tot = (t0 + t1) + (t2 + t3);
    out[col] = accumulate ? out[col] + tot : tot;
  }
  if (threadIdx.x == 0) tickets[blockIdx.x] = 0;
}

// Column sum of a bf16 matrix [rows, N] into partials[slice][N] (bias gradients).
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const __nv_bfloat16* __restrict__ a, int lda, float* __restrict__ part, int rows, int N,
                      int rows_per_slice) {
  __shared__ float sm[8][64];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + tx) * 2;
  const int r0 = blockIdx.y * rows_per_slice;
  const int r1 = min(rows, r0 + rows_per_slice);
  float s0 = 0.f, s1 = 0.f;
  if (col < N) {
    for (int r = r0 + ty; r < r1; r += 8) {
      const float2 d = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(a + static_cast<size_t>(r) * lda + col));
      s0 += d.x;
      s1 += d.y;
    }
  }
  sm[ty][tx * 2] = s0;
  sm[ty][tx * 2 + 1] = s1;
  __syncthreads();
  if (ty == 0 && col < N) {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      a0 += sm[k][tx * 2];
      a1 += sm[k][tx * 2 + 1];
    }
    part[static_cast<size_t>(blockIdx.y) * N + col] = a0;
    part[static_cast<size_t>(blockIdx.y) * N + col + 1] = a1;
  }
}

}  // namespace

int layernorm_fwd_launch(const void* x, const void* residual, const float* gamma, const float* beta, void* y,
                         void* sum_out, float* mean, float* rstd, int rows, int H, float eps, int num_sms,
                         cudaStream_t stream) {
  if (H % 8) return -3;
  const int blocks = min((rows + kLnWarpsPerBlock - 1) / kLnWarpsPerBlock, num_sms * 16);
  const dim3 grid(blocks), block(kLnWarpsPerBlock * 32);
  const auto* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  const auto* rb = reinterpret_cast<const __nv_bfloat16*>(residual);
  auto* yb = reinterpret_cast<__nv_bfloat16*>(y);
  auto* sb = reinterpret_cast<__nv_bfloat16*>(sum_out);
#define SSB_LN_CASE(V)                                                                                       \
  ln_fwd_kernel<V><<<grid, block, 0, stream>>>(xb, rb, gamma, beta, yb, sb, mean, rstd, rows, H, eps)
  switch (H) {
    case 512: SSB_LN_CASE(2); break;
    case 1024: SSB_LN_CASE(4); break;
    case 2048: SSB_LN_CASE(8); break;
    case 4096: SSB_LN_CASE(16); break;
    default: SSB_LN_CASE(0); break;
  }
#undef SSB_LN_CASE
  return static_cast<int>(cudaGetLastError());
}

// part_g / part_b: scratch of `slices` x H floats each (slices = ln_bwd_slices(rows)).
int ln_bwd_slices(int rows) {
  int s = (rows + 255) / 256;
  return s < 1 ? 1 : (s > 128 ? 128 : s);
}

// Rows of partial sums the backward needs in each of part_g / part_b (then H floats per row).
int ln_bwd_part_rows(int rows, int H, int num_sms) {
  if (H == 1024 || H == 2048) {  // one-pass kernel: one row of partials per block
    const int rpb = H == 1024 ? kLnWarpsPerBlock : kLnWarpsPerBlock / 2;   // rows a block works on at a time
    const int want = (rows + rpb - 1) / rpb;
    const int cap = num_sms * (H == 1024 ? 2 : 3);   // resident blocks per SM at the kernels' register counts
    return want < cap ? want : cap;
  }
  return ln_bwd_slices(rows);
}

int layernorm_bwd_launch(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                         const void* dres, void* dx, float* dgamma, float* dbeta, float* part_g, float* part_b,
                         int accumulate_wgrad, int rows, int H, int num_sms, cudaStream_t stream) {
  if (H % 8) return -3;
  const auto* dyb = reinterpret_cast<const __nv_bfloat16*>(dy);
  const auto* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  const auto* drb = reinterpret_cast<const __nv_bfloat16*>(dres);
  auto* dxb = reinterpret_cast<__nv_bfloat16*>(dx);
  if (H == 1024 || H == 2048) {
    // dy and x are read once: dx and the per-column sums come out of the same sweep
    const int nb = ln_bwd_part_rows(rows, H, num_sms);
    const dim3 g(nb), b(kLnWarpsPerBlock * 32);
    if (H == 1024)
      ln_bwd_onepass_kernel<4, 1><<<g, b, 0, stream>>>(dyb, xb, gamma, mean, rstd, drb, dxb, part_g, part_b, rows, H);
    else
      ln_bwd_onepass_kernel<4, 2><<<g, b, 0, stream>>>(dyb, xb, gamma, mean, rstd, drb, dxb, part_g, part_b, rows, H);
    fold_partials2_kernel<<<dim3((H + 63) / 64, 2), 256, 0, stream>>>(part_g, part_b, dgamma, dbeta, nb, H,
                                                                      accumulate_wgrad);
    return static_cast<int>(cudaGetLastError());
  }
  const int blocks = min((rows + kLnWarpsPerBlock - 1) / kLnWarpsPerBlock, num_sms * 16);
  const dim3 g(blocks), b(kLnWarpsPerBlock * 32);
  ln_bwd_dx_kernel<<<g, b, 0, stream>>>(dyb, xb, gamma, mean, rstd, drb, dxb, rows, H);
  const int slices = ln_bwd_slices(rows);
  const int rps = (rows + slices - 1) / slices;
  dim3 grid((H / 2 + 31) / 32, slices);
  ln_bwd_gb_partial_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dy),
                                                     reinterpret_cast<const __nv_bfloat16*>(x), mean, rstd, part_g,
                                                     part_b, rows, H, rps);
  fold_partials2_kernel<<<dim3((H + 63) / 64, 2), 256, 0, stream>>>(part_g, part_b, dgamma, dbeta, slices, H,
                                                                    accumulate_wgrad);
  return static_cast<int>(cudaGetLastError());
}

// out[N] (+)= column sums of a[rows, N]; `part` is scratch of ln_bwd_slices(rows) x N floats; `tickets` holds
// kColsumTickets zero-initialised counters that every call leaves at zero.
int colsum_launch(const void* a, int lda, float* out, float* part, int* tickets, int accumulate, int rows, int N,
                  cudaStream_t stream) {
  if (N % 2 || lda % 2) return -3;
  const int slices = ln_bwd_slices(rows);
  const int rps = (rows + slices - 1) / slices;
  const int colblocks = (N + 255) / 256;
  if (N % 8 == 0 && lda % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 && colblocks <= kColsumTickets &&
      tickets != nullptr) {
    // about eight blocks per SM in all, and never more slices than the scratch has rows
    int sl = (148 * 8 + colblocks - 1) / colblocks;
    sl = sl < 1 ? 1 : (sl > slices ? slices : sl);
    const int rows_per = (rows + sl - 1) / sl;
    colsum_onepass_kernel<<<dim3(colblocks, sl), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(a), lda, part,
                                                                   out, tickets, rows, N, rows_per, accumulate);
    return static_cast<int>(cudaGetLastError());
  }
  dim3 grid((N / 2 + 31) / 32, slices);
  colsum_partial_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(a), lda, part, rows, N, rps);
  fold_partials_kernel<<<(N + 255) / 256, 256, 0, stream>>>(part, out, slices, N, accumulate);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ssb
