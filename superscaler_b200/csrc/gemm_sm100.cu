// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory (128B swizzle)
// -> tcgen05.mma with fp32 accumulators in TMEM -> tcgen05.ld epilogue with fused
// bias / GeLU / dropout / residual / accumulate.
//
// Replaces the cuBLAS calls behind the reference's ColumnParallelLinear / RowParallelLinear
// (runtime/megatron/mpu/layers.py:363,459,532,593) and the TorchScript bias-gelu /
// bias-dropout-add fusions (runtime/megatron/model/fused_bias_gelu.py:31-45,
// runtime/megatron/model/flex_ops.py:61-83), which become epilogues here.
//
// CTA layout (192 threads, one CTA per SM, persistent over output tiles):
//   warp 0     : TMA producer (one elected lane)
//   warp 1     : TMEM allocator + MMA issuer (one elected lane)
//   warps 2..5 : epilogue; warp w reads TMEM lanes 32*(w%4) .. +31 (one output row per thread)
// Tile 128 x BN x 64, BN in {128, 256}; two accumulator stages of BN TMEM columns so the
// epilogue of tile i overlaps the main loop of tile i+1.
#include "common.cuh"
#include "gemm_sm100.cuh"
#include "gemm_epilogue.cuh"

namespace ssb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kGemmThreads = 192;
constexpr int kGroupM = 8;

template <int BN>
struct TileCfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;  // 512 or 256: powers of two >= 32
  // data + barriers + alignment slack
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

struct TileCoord {
  int m_blk, n_blk;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n) {
  const int per_group = kGroupM * num_n;
  const int group = tile / per_group;
  const int first_m = group * kGroupM;
  const int gsize = min(num_m - first_m, kGroupM);
  const int in_group = tile - group * per_group;
  TileCoord c;
  c.m_blk = first_m + in_group % gsize;
  c.n_blk = in_group / gsize;
  return c;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmParams p) {
  using Cfg = TileCfg<BN>;
  constexpr int kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * Cfg::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full_bar = bars + 2 * kStages;
  uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  // split-K: work item w = (slice, tile); slice s reduces the K blocks [s * kb_per, min(num_kb, (s + 1) * kb_per))
  const int splits = p.k_splits > 1 ? p.k_splits : 1;
  const int kb_per = (num_kb + splits - 1) / splits;
  const int num_work = num_tiles * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tmem_full_bar[s], 1);
      mbar_init(&tmem_empty_bar[s], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const TileCoord tc = tile_coord(w % num_tiles, num_m, num_n);
        const int kb0 = (w / num_tiles) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          uint8_t* sa = smem_a + stage * Cfg::kABytes;
          uint8_t* sb = smem_b + stage * Cfg::kBBytes;
          if (!A_MN) {
            tma_load_2d(sa, &tma_a, &full_bar[stage], kb * BK, tc.m_blk * BM);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (64 * BK * 2), &tma_a, &full_bar[stage], tc.m_blk * BM + c * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tma_b, &full_bar[stage], kb * BK, tc.n_blk * BN);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (64 * BK * 2), &tma_b, &full_bar[stage], tc.n_blk * BN + c * 64, kb * BK);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Unwinding: let the copies this thread already issued land before the CTA exits.
        for (int s = 0; s < kStages; ++s) {
          // A stage behind `stage` was last armed in the current phase, one at or after it in the previous one.
          const uint32_t armed_phase = (s < stage) ? phase : (phase ^ 1);
          for (uint32_t it = 0; it < (1u << 20); ++it)
            if (mbar_try_wait(&full_bar[s], armed_phase)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        const int kb0 = (w / num_tiles) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem_a + stage * Cfg::kABytes);
          const uint32_t sb = smem_u32(smem_b + stage * Cfg::kBBytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // K-major: 16 K elements = 32 bytes inside the 128-byte swizzled row.
            // MN-major: 16 K rows of 128 bytes; 64-element MN chunks are 64*BK*2 bytes apart.
            const uint64_t da = A_MN ? umma_desc_sw128(sa + k * 2048, 64 * BK * 2, 1024)
                                     : umma_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_desc_sw128(sb + k * 2048, 64 * BK * 2, 1024)
                                     : umma_desc_sw128(sb + k * 32, 16, 1024);
            umma_f16_ss(tmem_d, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tmem_full_bar[acc]);
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quarter = warp & 3;
    const uint32_t keep16 = dropout_keep16(p.dropout_p);
    const float drop_scale = p.dropout_p > 0.f ? 65536.0f / static_cast<float>(keep16) : 1.0f;
    int iter = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++iter) {
      const TileCoord tc = tile_coord(w % num_tiles, num_m, num_n);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row = tc.m_blk * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const int out_row = row + (w / num_tiles) * p.M;   // split-K: the output is the slice's [M, N] workspace block
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int n0 = tc.n_blk * BN + c * 32;
        if (n0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        gemm_epilogue_chunk<32>(p, out_row, n0, r, keep16, drop_scale);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
    }
  }

  // ------------------------------- teardown ----------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicMax(p.status, static_cast<int>(kStatusMbarTimeout));
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------ host side -----------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

}  // namespace

// bf16 row-major matrix [rows][cols] with leading dimension ld (elements): box = box_rows x 64 columns,
// 128-byte swizzle, zero fill outside the tensor.
int make_tma_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                     uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  // The encode call is a driver entry point: make sure this thread (e.g. an autograd worker that has made no
  // runtime call yet) has the device's primary context bound.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// fp32 row-major matrix [rows][cols] (contiguous rows): box = box_rows x 32 columns (128 bytes), 128-byte swizzle.
// Used as the destination of bulk tensor reductions (shared memory tile added to global memory).
int make_tma_2d_f32(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 4};
  cuuint32_t box[2] = {32, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

namespace {

// D[m][n] (+)= sum over the slices, in slice order, of ws[slice][m][n] (N a multiple of 4).
__global__ void __launch_bounds__(256)
splitk_fold_kernel(const float* __restrict__ ws, float* __restrict__ D, int ldd, int M, int N, int splits, int accumulate) {
  const int nq = N / 4;
  const long long quads = static_cast<long long>(M) * nq;
  const size_t slice = static_cast<size_t>(M) * N;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < quads; i += gridDim.x * 256LL) {
    const int m = static_cast<int>(i / nq), c = static_cast<int>(i % nq) * 4;
    const float* src = ws + static_cast<size_t>(m) * N + c;
    float4 acc = *reinterpret_cast<const float4*>(src);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(src + s * slice);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float4* dst = reinterpret_cast<float4*>(D + static_cast<size_t>(m) * ldd + c);
    if (accumulate) {
      const float4 o = *dst;
      acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
    }
    *dst = acc;
  }
}

template <int BN, bool A_MN, bool B_MN>
int launch_variant(const void* A, int lda, const void* B, int ldb, const GemmParams& p, int num_sms,
                   cudaStream_t stream) {
  using Cfg = TileCfg<BN>;
  CUtensorMap ta, tb;
  int rc;
  if (!A_MN)
    rc = make_tma_2d_bf16(&ta, A, p.M, p.K, lda, BM, BK);
  else
    rc = make_tma_2d_bf16(&ta, A, p.K, p.M, lda, BK, 64);
  if (rc != 0) return rc;
  if (!B_MN)
    rc = make_tma_2d_bf16(&tb, B, p.N, p.K, ldb, BN, BK);
  else
    rc = make_tma_2d_bf16(&tb, B, p.K, p.N, ldb, BK, 64);
  if (rc != 0) return rc;

  auto kernel = gemm_bf16_kernel<BN, A_MN, B_MN>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done = true;
  }
  const int num_tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  if (p.k_splits > 1) {
    // every slice writes a plain fp32 [M, N] block of the workspace; the fold adds them, in slice order, into D
    GemmParams q = p;
    q.D = p.split_ws;
    q.ldd = p.N;
    q.out_fp32 = 1;
    q.accumulate = 0;
    const int work = num_tiles * p.k_splits;
    kernel<<<work < num_sms ? work : num_sms, kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, q);
    const long long quads = static_cast<long long>(p.M) * (p.N / 4);
    const int blocks = static_cast<int>((quads + 255) / 256 < num_sms * 8LL ? (quads + 255) / 256 : num_sms * 8LL);
    splitk_fold_kernel<<<blocks, 256, 0, stream>>>(p.split_ws, reinterpret_cast<float*>(p.D), p.ldd, p.M, p.N, p.k_splits,
                                                   p.accumulate);
    return static_cast<int>(cudaGetLastError());
  }
  const int grid = num_tiles < num_sms ? num_tiles : num_sms;
  kernel<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

int gemm2_bf16_launch(const void* A, int lda, int a_mn_major, const void* B, int ldb, int b_mn_major,
                      const GemmParams& p, int num_sms, cudaStream_t stream);

// 0 = always the one-CTA kernel, 1 = two-SM kernel where the output has enough 256 x 256 tiles.
static int g_pair_mode = 1;
void gemm_set_pair_mode(int mode) { g_pair_mode = mode; }
int gemm_get_pair_mode() { return g_pair_mode; }

int gemm_splitk_splits(int M, int N, int K, int num_sms) {
  if (g_pair_mode) {
    const int tiles_pair = ((M + 255) / 256) * ((N + 255) / 256);
    if (M >= 256 && N >= 256 && tiles_pair >= num_sms / 4) return 1;     // the two-SM kernel takes it
  }
  if (N % 4) return 1;
  const int tiles256 = ((M + BM - 1) / BM) * ((N + 255) / 256);
  const bool bn128 = (N <= 128) || (tiles256 < num_sms);
  const int tiles = ((M + BM - 1) / BM) * ((N + (bn128 ? 127 : 255)) / (bn128 ? 128 : 256));
  const int num_kb = (K + BK - 1) / BK;
  int s = num_sms / tiles;                 // slices until every SM has a work item
  if (s > num_kb / 16) s = num_kb / 16;    // at least 16 K blocks (1024 reduction steps) per slice
  if (s > 64) s = 64;
  if (s < 2) return 1;
  const int kb_per = (num_kb + s - 1) / s;
  return (num_kb + kb_per - 1) / kb_per;   // no empty slice
}

// Launches the GEMM on `stream`.  Returns 0 or a CUDA / driver error code; argument errors are negative.
int gemm_bf16_launch(const void* A, int lda, int a_mn_major, const void* B, int ldb, int b_mn_major,
                     const GemmParams& p, int num_sms, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) return -2;
  if ((lda % 8) || (ldb % 8) || (p.ldd % (p.out_fp32 ? 4 : 8))) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(p.D) & 15))
    return -4;
  if (p.k_splits > 1) {
    const bool plain = p.out_fp32 && p.alpha == 1.0f && p.bias == nullptr && p.act == 0 && p.aux == nullptr &&
                       p.preact_out == nullptr && p.residual == nullptr && p.dropout_p == 0.f;
    if (!plain || p.split_ws == nullptr || (p.N % 4) || (reinterpret_cast<uintptr_t>(p.split_ws) & 15) ||
        p.k_splits > (p.K + BK - 1) / BK)
      return -5;
  } else if (g_pair_mode) {
    const int tiles_pair = ((p.M + 255) / 256) * ((p.N + 255) / 256);
    if (p.M >= 256 && p.N >= 256 && tiles_pair >= num_sms / 4)
      return gemm2_bf16_launch(A, lda, a_mn_major, B, ldb, b_mn_major, p, num_sms, stream);
  }
  // Narrow outputs use the 128-wide tile so fewer columns are wasted and more CTAs are busy.
  const int tiles256 = ((p.M + BM - 1) / BM) * ((p.N + 255) / 256);
  const bool bn128 = (p.N <= 128) || (tiles256 < num_sms);
  if (!a_mn_major && !b_mn_major)
    return bn128 ? launch_variant<128, false, false>(A, lda, B, ldb, p, num_sms, stream)
                 : launch_variant<256, false, false>(A, lda, B, ldb, p, num_sms, stream);
  if (!a_mn_major && b_mn_major)
    return bn128 ? launch_variant<128, false, true>(A, lda, B, ldb, p, num_sms, stream)
                 : launch_variant<256, false, true>(A, lda, B, ldb, p, num_sms, stream);
  if (a_mn_major && b_mn_major)
    return bn128 ? launch_variant<128, true, true>(A, lda, B, ldb, p, num_sms, stream)
                 : launch_variant<256, true, true>(A, lda, B, ldb, p, num_sms, stream);
  return bn128 ? launch_variant<128, true, false>(A, lda, B, ldb, p, num_sms, stream)
               : launch_variant<256, true, false>(A, lda, B, ldb, p, num_sms, stream);
}

}  // namespace ssb
