// Epilogue of the tcgen05 GEMM family for one thread: W consecutive output columns [n0, n0+W) of row `row`
// (W = 16 or 32, n0 a multiple of W), accumulators in r (fp32 bit patterns).  Order of operations: see GemmParams.
// All operands are read and written in 16-byte pieces when the whole chunk lies inside the matrix.
#pragma once
#include "common.cuh"
#include "gemm_sm100.cuh"

namespace ssb {

// 8 bf16 values <-> 8 floats
__device__ __forceinline__ void unpack8(const uint4 q, float* f) {
  float2 t;
  t = unpack_bf16x2(q.x); f[0] = t.x; f[1] = t.y;
  t = unpack_bf16x2(q.y); f[2] = t.x; f[3] = t.y;
  t = unpack_bf16x2(q.z); f[4] = t.x; f[5] = t.y;
  t = unpack_bf16x2(q.w); f[6] = t.x; f[7] = t.y;
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]);
  q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]);
  q.w = pack_bf16x2(f[6], f[7]);
  return q;
}

template <int W>
__device__ __forceinline__ void gemm_epilogue_chunk(const GemmParams& p, int row, int n0, const uint32_t (&r)[W],
                                                    uint32_t keep16, float drop_scale) {
  static_assert(W == 16 || W == 32, "chunk width");
  float v[W];
#pragma unroll
  for (int i = 0; i < W; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
  const bool full = (n0 + W <= p.N);

  if (p.bias != nullptr) {
    if (p.bias_fp32) {
      const float* b = reinterpret_cast<const float*>(p.bias) + n0;
      if (full) {
#pragma unroll
        for (int i = 0; i < W / 4; ++i) {
          const float4 q = __ldg(reinterpret_cast<const float4*>(b) + i);
          v[4 * i] += q.x; v[4 * i + 1] += q.y; v[4 * i + 2] += q.z; v[4 * i + 3] += q.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < W; ++i)
          if (n0 + i < p.N) v[i] += __ldg(b + i);
      }
    } else {
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + n0;
      if (full) {
#pragma unroll
        for (int i = 0; i < W / 8; ++i) {
          float f[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(b) + i), f);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[8 * i + e] += f[e];
        }
      } else {
#pragma unroll
        for (int i = 0; i < W; ++i)
          if (n0 + i < p.N) v[i] += __bfloat162float(b[i]);
      }
    }
  }
  if (p.preact_out != nullptr) {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.preact_out) + static_cast<size_t>(row) * p.ldpre + n0;
    if (full) {
#pragma unroll
      for (int i = 0; i < W / 8; ++i) reinterpret_cast<uint4*>(o)[i] = pack8(v + 8 * i);
    } else {
      for (int i = 0; i < W && n0 + i < p.N; ++i) o[i] = __float2bfloat16(v[i]);
    }
  }
  if (p.act == kActGelu) {
#pragma unroll
    for (int i = 0; i < W; ++i) v[i] = gelu_tanh(v[i]);
  } else if (p.act == kActRelu) {
#pragma unroll
    for (int i = 0; i < W; ++i) v[i] = fmaxf(v[i], 0.f);
  } else if (p.act == kActDGelu || p.act == kActDRelu) {
    const __nv_bfloat16* a =
        reinterpret_cast<const __nv_bfloat16*>(p.aux) + static_cast<size_t>(row) * p.ldaux + n0;
    float x[W];
    if (full) {
#pragma unroll
      for (int i = 0; i < W / 8; ++i) unpack8(__ldg(reinterpret_cast<const uint4*>(a) + i), x + 8 * i);
    } else {
#pragma unroll
      for (int i = 0; i < W; ++i) x[i] = (n0 + i < p.N) ? __bfloat162float(a[i]) : 0.f;
    }
    if (p.act == kActDGelu) {
#pragma unroll
      for (int i = 0; i < W; ++i) v[i] *= gelu_tanh_grad(x[i]);
    } else {
#pragma unroll
      for (int i = 0; i < W; ++i) v[i] = x[i] > 0.f ? v[i] : 0.f;
    }
  }
  if (p.dropout_p > 0.f) {
    // flat index = row * N + col; groups of 4 consecutive columns (n0 is a multiple of 16)
    const uint64_t g0 = (static_cast<uint64_t>(row) * static_cast<uint64_t>(p.N) + n0) >> 2;
#pragma unroll
    for (int g = 0; g < W / 4; ++g) {
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
      for (int i = 0; i < W / 8; ++i) {
        float f[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(a) + i), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[8 * i + e] += f[e];
      }
    } else {
      for (int i = 0; i < W && n0 + i < p.N; ++i) v[i] += __bfloat162float(a[i]);
    }
  }
  if (p.out_fp32) {
    float* o = reinterpret_cast<float*>(p.D) + static_cast<size_t>(row) * p.ldd + n0;
    if (full) {
#pragma unroll
      for (int i = 0; i < W / 4; ++i) {
        float4 q = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        if (p.accumulate) {
          const float4 old = reinterpret_cast<const float4*>(o)[i];
          q.x += old.x; q.y += old.y; q.z += old.z; q.w += old.w;
        }
        reinterpret_cast<float4*>(o)[i] = q;
      }
    } else {
      for (int i = 0; i < W && n0 + i < p.N; ++i) o[i] = p.accumulate ? o[i] + v[i] : v[i];
    }
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<size_t>(row) * p.ldd + n0;
    if (full) {
#pragma unroll
      for (int i = 0; i < W / 8; ++i) {
        if (p.accumulate) {
          float f[8];
          unpack8(reinterpret_cast<const uint4*>(o)[i], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[8 * i + e] += f[e];
        }
        reinterpret_cast<uint4*>(o)[i] = pack8(v + 8 * i);
      }
    } else {
      for (int i = 0; i < W && n0 + i < p.N; ++i) {
        float w = v[i];
        if (p.accumulate) w += __bfloat162float(o[i]);
        o[i] = __float2bfloat16(w);
      }
    }
  }
}

// Arithmetic part of the epilogue for 16 columns when the row operands (derivative input `aux` or `residual`) have
// already been brought on chip: v = epilogue(acc) with the same order of operations as gemm_epilogue_chunk.
// `operand` holds the 16 bf16 values of aux (for the derivative activations) or of the residual, or is unused.
__device__ __forceinline__ void gemm_epilogue_math16(const GemmParams& p, int row, int n0, const uint32_t (&r)[16],
                                                     const uint4 (&operand)[2], uint32_t keep16, float drop_scale,
                                                     float (&pre)[16], float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
  if (p.bias != nullptr) {
    if (p.bias_fp32) {
      const float* b = reinterpret_cast<const float*>(p.bias) + n0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(b) + i);
        v[4 * i] += q.x; v[4 * i + 1] += q.y; v[4 * i + 2] += q.z; v[4 * i + 3] += q.w;
      }
    } else {
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + n0;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float f[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(b) + i), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[8 * i + e] += f[e];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) pre[i] = v[i];
  float x[16];
  if (p.act == kActDGelu || p.act == kActDRelu || p.residual != nullptr) {
    unpack8(operand[0], x);
    unpack8(operand[1], x + 8);
  }
  if (p.act == kActGelu) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = gelu_tanh(v[i]);
  } else if (p.act == kActRelu) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i], 0.f);
  } else if (p.act == kActDGelu) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] *= gelu_tanh_grad(x[i]);
  } else if (p.act == kActDRelu) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = x[i] > 0.f ? v[i] : 0.f;
  }
  if (p.dropout_p > 0.f) {
    const uint64_t g0 = (static_cast<uint64_t>(row) * static_cast<uint64_t>(p.N) + n0) >> 2;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint32_t m = dropout_keep4(p.dropout_seed, g0 + g, keep16);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[4 * g + i] = ((m >> i) & 1u) ? v[4 * g + i] * drop_scale : 0.f;
    }
  }
  if (p.residual != nullptr) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] += x[i];
  }
}

}  // namespace ssb
