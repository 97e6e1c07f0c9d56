// All-gather fused into the GEMM that consumes it, in ONE persistent kernel over peer memory.
//
//   Y = epilogue( concat over tp ranks r of X_r  .  W^T )        X_r : this rank's rows [M/tp, K],  W : [N, K]
//
// Replaces "all-gather the activation, then run the column-parallel GEMM" (the gather half of the reference's
// tensor_adapter / _PrimReplicate, runtime/megatron/mpu/mappings.py:273-286,382-468, followed by
// ColumnParallelLinear, runtime/megatron/mpu/layers.py:459-470): there the GEMM starts only after the whole gather.
//
//   warp 0      TMA producer: output tiles are ordered so that the m-blocks of this rank's OWN rows come first (read
//               straight from X_r), then the rows of rank+1, rank+2, ... (read from the local gather buffer, each
//               m-block only after its "arrived" flag is set)
//   warp 1      TMEM allocator + MMA issuer
//   warps 2..5  epilogue (bias / activation / dropout / residual, as gemm_bf16_kernel)
//   warp 6      pusher: copies this rank's rows, one 128-row m-block at a time (CTA c takes m-blocks c, c + grid, ...),
//               from X_r through a double-buffered 16 KB staging area in shared memory (bulk load, then one bulk
//               store per peer) into the same rows of every peer's gather buffer, then release-stores the m-block's
//               flag on every peer.  Each remote row crosses NVLink once per peer; the tiles that need it read the
//               local copy.
//
// No TMA load ever reads a peer's memory and nothing is multicast.  Gather buffers alternate between two
// allocations by call parity: a rank that is one call ahead pushes into the buffer its peers are not reading.
// Flags carry a growing epoch and are never reset; every wait is bounded (kStatusPeerTimeout on expiry).
#include <cuda.h>

#include "common.cuh"
#include "gemm_ag_sm100.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_sm100.cuh"

namespace ssb {

int make_tma_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                     uint32_t box_rows, uint32_t box_cols);

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kThreads = 64 + 128 + 32;
constexpr int kABytes = BM * BK * 2, kBBytes = BN * BK * 2, kStageBytes = kABytes + kBBytes;
constexpr int kPushChunk = 16384;                   // bytes per staged piece
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kPushChunk + 1024 + 256;
constexpr int kGroupM = 8;
constexpr uint64_t kPeerLimitNs = 20ull * 1000 * 1000 * 1000;

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// global -> shared bulk copy, completion counted in bytes on an mbarrier of this CTA
__device__ __forceinline__ void bulk_copy_g2s(void* sdst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(sdst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_copy_s2g(void* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Bounded wait (one thread) until *flag >= epoch.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, volatile int* abort_flag, int* status) {
  uint64_t t0 = 0;
  for (uint32_t it = 0; it < (1u << 30); ++it) {
    if (ld_acquire_sys_u32(flag) >= epoch) return true;
    if ((it & 1023u) == 1023u) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kPeerLimitNs) break;
    }
  }
  *abort_flag = 1;
  if (status != nullptr) atomicMax(status, static_cast<int>(kStatusPeerTimeout));
  return false;
}

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

__global__ void __launch_bounds__(kThreads, 1)
gemm_ag_kernel(const __grid_constant__ CUtensorMap tma_local, const __grid_constant__ CUtensorMap tma_gather,
               const __grid_constant__ CUtensorMap tma_b, const GemmParams p, const GemmAgComm cm) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kABytes;
  uint8_t* push_buf = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(push_buf + 2 * kPushChunk);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full_bar = bars + 2 * kStages;
  uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;
  uint64_t* push_bar = bars + 2 * kStages + 4;  // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = p.M / BM;                  // M = tp * rows_per_rank, rows_per_rank a multiple of 128
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int mb_per_rank = num_m / cm.tp;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tmem_full_bar[s], 1);
      mbar_init(&tmem_empty_bar[s], 4);
      mbar_init(&push_bar[s], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tma_local);
    tma_prefetch_desc(&tma_gather);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // logical m-block i (the order tiles are computed in) -> source rank and global m-block
  auto src_of = [&](int i) { return (cm.rank + i / mb_per_rank) % cm.tp; };
  auto mblk_of = [&](int i) { return src_of(i) * mb_per_rank + i % mb_per_rank; };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t* my_flags = cm.flag_ptrs[cm.rank];
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, num_m, num_n);
        const int src = src_of(tc.m_blk);
        const int m_blk = mblk_of(tc.m_blk);
        const bool local = src == cm.rank;
        if (!local) {
          // rows pushed by rank `src`: wait for their flag, then make them visible to the TMA (async proxy) reads
          if (!wait_flag(my_flags + m_blk, cm.epoch, abort_flag, p.status)) { ok = false; break; }
          fence_proxy_async_global();
        }
        const CUtensorMap* ta = local ? &tma_local : &tma_gather;
        const int row = local ? (m_blk - cm.rank * mb_per_rank) * BM : m_blk * BM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
          tma_load_2d(smem_a + stage * kABytes, ta, &full_bar[stage], kb * BK, row);
          tma_load_2d(smem_b + stage * kBBytes, &tma_b, &full_bar[stage], kb * BK, tc.n_blk * BN);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        for (int s = 0; s < kStages; ++s) {
          const uint32_t armed_phase = (s < stage) ? phase : (phase ^ 1);
          for (uint32_t it = 0; it < (1u << 20); ++it)
            if (mbar_try_wait(&full_bar[s], armed_phase)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, false, false);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++iter) {
        const int acc = iter & 1;
        if (!mbar_wait(&tmem_empty_bar[acc], ((iter >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem_a + stage * kABytes);
          const uint32_t sb = smem_u32(smem_b + stage * kBBytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_f16_ss(tmem_d, umma_desc_sw128(sa + k * 32, 16, 1024), umma_desc_sw128(sb + k * 32, 16, 1024), idesc,
                        (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full_bar[acc]);
      }
    }
  } else if (warp < 6) {
    // -------------------------------- epilogue --------------------------------
    const int quarter = warp & 3;
    const uint32_t keep16 = dropout_keep16(p.dropout_p);
    const float drop_scale = p.dropout_p > 0.f ? 65536.0f / static_cast<float>(keep16) : 1.0f;
    int iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++iter) {
      const TileCoord tc = tile_coord(tile, num_m, num_n);
      const int acc = iter & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full_bar[acc], (iter >> 1) & 1, abort_flag))) { ok = false; break; }
      tc_fence_after_sync();
      const int row = mblk_of(tc.m_blk) * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int n0 = tc.n_blk * BN + c * 32;
        if (n0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        gemm_epilogue_chunk<32>(p, row, n0, r, keep16, drop_scale);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
    }
  } else {
    // --------------------------------- pusher ---------------------------------
    if (lane == 0 && cm.tp > 1) {
      const size_t row_bytes = static_cast<size_t>(p.K) * 2;              // X_r and the gather buffers are dense
      const size_t blk_bytes = static_cast<size_t>(BM) * row_bytes;
      const uint8_t* x = reinterpret_cast<const uint8_t*>(cm.x_local);
      const int pieces_per_blk = static_cast<int>(blk_bytes / kPushChunk);
      int my_blocks = 0;
      for (int b = blockIdx.x; b < mb_per_rank; b += gridDim.x) ++my_blocks;
      const int total = my_blocks * pieces_per_blk;
      // piece j (of this CTA) lives in buffer j & 1 and completes phase (j >> 1) & 1 of that buffer's barrier
      auto src_ptr = [&](int j) {
        const int b = blockIdx.x + (j / pieces_per_blk) * gridDim.x;
        return x + static_cast<size_t>(b) * blk_bytes + static_cast<size_t>(j % pieces_per_blk) * kPushChunk;
      };
      auto issue_load = [&](int j) {
        mbar_arrive_expect_tx(&push_bar[j & 1], kPushChunk);
        bulk_copy_g2s(push_buf + (j & 1) * kPushChunk, src_ptr(j), kPushChunk, &push_bar[j & 1]);
      };
      bool ok = true;
      if (total > 0) issue_load(0);
      for (int j = 0; j < total && ok; ++j) {
        if (j + 1 < total) {
          tma_store_wait_read<0>();  // the stores of piece j - 1 have left the other buffer
          issue_load(j + 1);
        }
        if (!mbar_wait(&push_bar[j & 1], (j >> 1) & 1, abort_flag)) { ok = false; break; }
        const int b = blockIdx.x + (j / pieces_per_blk) * gridDim.x;
        const size_t dst_off = (static_cast<size_t>(cm.rank) * mb_per_rank + b) * blk_bytes +
                               static_cast<size_t>(j % pieces_per_blk) * kPushChunk;
        for (int pr = 0; pr < cm.tp; ++pr)
          if (pr != cm.rank)
            bulk_copy_s2g(reinterpret_cast<uint8_t*>(cm.gather_ptrs[pr]) + dst_off, push_buf + (j & 1) * kPushChunk,
                          kPushChunk);
        tma_store_commit();
        if (j % pieces_per_blk == pieces_per_blk - 1) {
          tma_store_wait<0>();  // the whole m-block has been written on every peer
          for (int pr = 0; pr < cm.tp; ++pr)
            if (pr != cm.rank) st_release_sys_u32(cm.flag_ptrs[pr] + cm.rank * mb_per_rank + b, cm.epoch);
        }
      }
      if (!ok) {  // let the load in flight land before the CTA exits
        for (uint32_t it = 0; it < (1u << 20); ++it)
          if (mbar_try_wait(&push_bar[0], 0) || mbar_try_wait(&push_bar[0], 1)) break;
      }
      tma_store_wait<0>();
    }
  }

  // ------------------------------- teardown ----------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicMax(p.status, static_cast<int>(kStatusMbarTimeout));
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

}  // namespace

// x_local: this rank's rows [M / tp][K] bf16, dense.  W: [N][K] bf16 (K contiguous).  p.M is the gathered row count
// (tp x rows per rank, rows per rank a multiple of 128); p describes the epilogue and the local output [M][N].
// K must be a multiple of 64 and the rows of a 128-row block (128 x K x 2 bytes) a multiple of 16 KB.
int gemm2_ag_launch(const void* W, int ldw, const GemmParams& p, const GemmAgComm& cm, int num_sms, cudaStream_t stream);

int gemm_ag_launch(const void* W, int ldw, const GemmParams& p, const GemmAgComm& cm, int num_sms, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0 || p.K <= 0 || cm.tp < 1 || cm.tp > 32) return -2;
  if (p.M % (BM * cm.tp) || (p.K % 64) || (ldw % 8)) return -3;
  if (static_cast<long long>(p.M) * p.K > cm.capacity_elems || p.M / BM > cm.max_blocks) return -6;
  {  // large shapes run on the two-SM kernel
    const int rc2 = gemm2_ag_launch(W, ldw, p, cm, num_sms, stream);
    if (rc2 != -100) return rc2;
  }
  const int rows_local = p.M / cm.tp;
  CUtensorMap tl, tg, tb;
  int rc = make_tma_2d_bf16(&tl, cm.x_local, rows_local, p.K, p.K, BM, BK);
  if (rc != 0) return rc;
  rc = make_tma_2d_bf16(&tg, cm.gather_ptrs_host_local, p.M, p.K, p.K, BM, BK);
  if (rc != 0) return rc;
  rc = make_tma_2d_bf16(&tb, W, p.N, p.K, ldw, BN, BK);
  if (rc != 0) return rc;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_ag_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done = true;
  }
  const int num_tiles = (p.M / BM) * ((p.N + BN - 1) / BN);
  const int grid = num_tiles < num_sms ? num_tiles : num_sms;
  gemm_ag_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tl, tg, tb, p, cm);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ssb
