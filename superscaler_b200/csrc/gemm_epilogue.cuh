// Epilogue of the tcgen05 GEMM family for one thread: 32 consecutive output columns [n0, n0+32) of row `row`,
// accumulators in r (fp32 bit patterns).  Order of operations: see GemmParams.
#pragma once
#include "common.cuh"
#include "gemm_sm100.cuh"

namespace ssb {

__device__ __forceinline__ void gemm_epilogue_chunk(const GemmParams& p, int row, int n0, const uint32_t (&r)[32],
                                                    uint32_t keep16, float drop_scale) {
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
  const bool full = (n0 + 32 <= p.N);

  if (p.bias != nullptr) {
    if (p.bias_fp32) {
      const float* b = reinterpret_cast<const float*>(p.bias) + n0;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (full || n0 + i < p.N) v[i] += __ldg(b + i);
    } else {
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + n0;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (full || n0 + i < p.N) v[i] += __bfloat162float(b[i]);
    }
  }
  if (p.preact_out != nullptr) {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.preact_out) + static_cast<size_t>(row) * p.ldpre + n0;
    if (full) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 q;
        q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
        q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
        q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
        q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
        reinterpret_cast<uint4*>(o)[i] = q;
      }
    } else {
      for (int i = 0; i < 32 && n0 + i < p.N; ++i) o[i] = __float2bfloat16(v[i]);
    }
  }
  if (p.act == kActGelu) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
  } else if (p.act == kActRelu) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.f);
  } else if (p.act == kActDGelu || p.act == kActDRelu) {
    const __nv_bfloat16* a =
        reinterpret_cast<const __nv_bfloat16*>(p.aux) + static_cast<size_t>(row) * p.ldaux + n0;
    float x[32];
    if (full) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(a) + i);
        float2 f;
        f = unpack_bf16x2(q.x); x[8 * i + 0] = f.x; x[8 * i + 1] = f.y;
        f = unpack_bf16x2(q.y); x[8 * i + 2] = f.x; x[8 * i + 3] = f.y;
        f = unpack_bf16x2(q.z); x[8 * i + 4] = f.x; x[8 * i + 5] = f.y;
        f = unpack_bf16x2(q.w); x[8 * i + 6] = f.x; x[8 * i + 7] = f.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) x[i] = (n0 + i < p.N) ? __bfloat162float(a[i]) : 0.f;
    }
    if (p.act == kActDGelu) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] *= gelu_tanh_grad(x[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = x[i] > 0.f ? v[i] : 0.f;
    }
  }
  if (p.dropout_p > 0.f) {
    // flat index = row * N + col; groups of 4 consecutive columns (n0 is a multiple of 32)
    const uint64_t g0 = (static_cast<uint64_t>(row) * static_cast<uint64_t>(p.N) + n0) >> 2;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const uint32_t m = dropout_keep4(p.dropout_seed, g0 + g, keep16);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[4 * g + i] = ((m >> i) & 1u) ? v[4 * g + i] * drop_scale : 0.f;
    }
  }
  if (p.residual != nullptr) {
    const __nv_bfloat16* a =
        reinterpret_cast<const __nv_bfloat16*>(p.residual) + static_cast<size_t>(row) * p.ldres + n0;
    if (full) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(a) + i);
        float2 f;
        f = unpack_bf16x2(q.x); v[8 * i + 0] += f.x; v[8 * i + 1] += f.y;
        f = unpack_bf16x2(q.y); v[8 * i + 2] += f.x; v[8 * i + 3] += f.y;
        f = unpack_bf16x2(q.z); v[8 * i + 4] += f.x; v[8 * i + 5] += f.y;
        f = unpack_bf16x2(q.w); v[8 * i + 6] += f.x; v[8 * i + 7] += f.y;
      }
    } else {
      for (int i = 0; i < 32 && n0 + i < p.N; ++i) v[i] += __bfloat162float(a[i]);
    }
  }
  if (p.out_fp32) {
    float* o = reinterpret_cast<float*>(p.D) + static_cast<size_t>(row) * p.ldd + n0;
    if (full) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 q = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        if (p.accumulate) {
          const float4 old = reinterpret_cast<const float4*>(o)[i];
          q.x += old.x; q.y += old.y; q.z += old.z; q.w += old.w;
        }
        reinterpret_cast<float4*>(o)[i] = q;
      }
    } else {
      for (int i = 0; i < 32 && n0 + i < p.N; ++i) o[i] = p.accumulate ? o[i] + v[i] : v[i];
    }
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<size_t>(row) * p.ldd + n0;
    if (full) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (p.accumulate) {
          const uint4 old = reinterpret_cast<const uint4*>(o)[i];
          float2 f;
          f = unpack_bf16x2(old.x); v[8 * i + 0] += f.x; v[8 * i + 1] += f.y;
          f = unpack_bf16x2(old.y); v[8 * i + 2] += f.x; v[8 * i + 3] += f.y;
          f = unpack_bf16x2(old.z); v[8 * i + 4] += f.x; v[8 * i + 5] += f.y;
          f = unpack_bf16x2(old.w); v[8 * i + 6] += f.x; v[8 * i + 7] += f.y;
        }
        uint4 q;
        q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
        q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
        q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
        q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
        reinterpret_cast<uint4*>(o)[i] = q;
      }
    } else {
      for (int i = 0; i < 32 && n0 + i < p.N; ++i) {
        float w = v[i];
        if (p.accumulate) w += __bfloat162float(o[i]);
        o[i] = __float2bfloat16(w);
      }
    }
  }
}

}  // namespace ssb
