// Device helpers shared by the tcgen05 flash-attention kernels (forward, the two-kernel backward and the fused
// backward): thread layout constants, the stateless dropout mask, swizzled shared-memory row stores and the
// warp-uniform bounded wait.
#pragma once

#include "attention_sm100.cuh"
#include "common.cuh"

namespace ssb {
namespace attn {

constexpr int kMathThreads = 512;               // 4 column groups x 4 warps
constexpr int kMathWarps = kMathThreads / 32;
constexpr int kAttnThreads = 64 + kMathThreads;  // + TMA warp + MMA warp
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t fmix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x85EBCA6Bu;
  x ^= x >> 13;
  x *= 0xC2B2AE35u;
  x ^= x >> 16;
  return x;
}
// Dropout mask: one 32-bit hash decides the four QUERIES 4t .. 4t+3 of one key; query 4t+i is kept when byte i of the
// hash is below keep8 = round(256 (1 - p)).  The dropout probability is therefore quantised to 1/256 (the scale
// applied to the kept values is the exact 256 / keep8), which makes the mask four times cheaper to generate than
// one 16-bit lane per element.  The backward kernels hold one KEY per thread and sixteen consecutive queries, so
// four hashes per thread cover a tile step without any exchange (the backward does 2.5 times the work of the
// forward); the kernels that hold one QUERY per thread share the hashes of a key between the four lanes of a
// query quad with shuffles.
__device__ __forceinline__ uint32_t attn_col_hash(uint32_t bh_seed, uint32_t key, uint32_t qquads, uint32_t qquad) {
  return fmix32((key * qquads + qquad) * 0x9E3779B1u + bh_seed);
}
__device__ __forceinline__ bool keep_byte(uint32_t h, int i, uint32_t keep8) { return ((h >> (8 * i)) & 0xFFu) < keep8; }
__host__ __device__ __forceinline__ uint32_t dropout_keep8(float p) {
  const int k = static_cast<int>((1.0f - p) * 256.0f + 0.5f);
  return static_cast<uint32_t>(k < 1 ? 1 : (k > 256 ? 256 : k));
}

// Writes 32 consecutive bf16 columns (16 packed words) of row r into a [rows][128 B] swizzled chunk.
// piece0 = index of the first 16-byte piece inside the 128-byte row (0 or 4).
__device__ __forceinline__ void store_row32_sw128(uint8_t* chunk, int r, int piece0, const uint32_t (&w)[16]) {
  uint8_t* row = chunk + r * 128;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int piece = (piece0 + i) ^ (r & 7);
    *reinterpret_cast<uint4*>(row + piece * 16) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
  }
}

// Writes 16 consecutive bf16 columns (8 packed words) of row r; piece0 = first 16-byte piece (even).
__device__ __forceinline__ void store_row16_sw128(uint8_t* chunk, int r, int piece0, const uint32_t (&w)[8]) {
  uint8_t* row = chunk + r * 128;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int piece = (piece0 + i) ^ (r & 7);
    *reinterpret_cast<uint4*>(row + piece * 16) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
  }
}

// Bounded wait whose outcome is the same for every lane of the warp, so that the warp-collective
// tcgen05.ld that follows is never executed by a part of the warp only.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}

// One arrival per warp on an mbarrier whose expected count is the number of warps: every lane has issued its fences,
// the warp converges, lane 0 arrives.  Five hundred arrivals on one shared-memory word serialise; sixteen do not.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

struct Pipe {
  int stage = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int n) {
    if (++stage == n) {
      stage = 0;
      phase ^= 1;
    }
  }
};


template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[N]) {
  if constexpr (N == 32) tmem_ld_32x32(taddr, r);
  else tmem_ld_32x16(taddr, r);
}

}  // namespace attn
}  // namespace ssb
