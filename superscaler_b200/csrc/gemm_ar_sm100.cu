// GEMM fused with the tensor-parallel all-reduce that follows it, in ONE persistent kernel over peer memory.
//
//   out = epilogue( sum over tp ranks r of  A_r . B_r^T )       (every rank ends up with the full `out`)
//
// Replaces RowParallelLinear.forward = F.linear + torch.distributed.all_reduce and the all-reduce of the
// input gradient of ColumnParallelLinear (runtime/megatron/mpu/layers.py:359,459-470,
// runtime/megatron/mpu/mappings.py:23-40 of the reference), which run the GEMM to completion and only then start
// the collective.  Here the reduction of output tile t overlaps the tensor-core work of tile t+1:
//
//   warp 0      TMA producer                         (as in gemm_bf16_kernel)
//   warp 1      TMEM allocator + MMA issuer
//   warps 2..5  partial epilogue: accumulator -> bf16 -> a 2 KB staging buffer in shared memory -> bulk asynchronous
//               copy (cp.async.bulk shared -> global) into the scratch of the tile's OWNER rank (tile % tp; the
//               owner's own partial goes the same way into local memory), then one release-store per
//               (tile, 32-row quarter) into the owner's flag table
//   warps 6..9  owner role: for a tile this rank owns, wait until every rank's partial quarter is flagged, add the
//               tp partial tiles (all local by now), apply bias / dropout / residual, write the rows to the local
//               output, stage them in shared memory and bulk-copy them into every peer's result buffer, then flag
//               the quarter as final on every peer
//   warps 10..13 receiver role: for a tile owned by a peer, wait for that flag and copy the rows from the local
//               result buffer into the local output.  (Two separate warp sets: with one set the ranks took turns,
//               each waiting for the other's owner work before starting its own.)
//
// Everything that crosses NVLink is a bulk copy issued to the copy engine of the SM followed by a flag: no warp
// waits for a remote load, and the load/store unit never queues remote stores.  (Measured on two B200: the same
// kernel with ordinary remote stores, or with remote loads, took GEMM time PLUS transfer time, because remote
// accesses queued in the load/store unit delay the local stores of the epilogue warps.)
// Traffic per rank is the two-shot optimum, 2 (tp-1)/tp x M x N x 2 bytes.
// There is no grid-wide or cross-rank barrier: a rank leaves the kernel only after it received every tile it does
// not own, i.e. after every owner finished reading this rank's partials; results alternate between two buffers
// so that an owner that is one call ahead never overwrites rows a peer is still copying.  Flags carry a
// monotonically growing epoch, so they are never reset.  Every wait is bounded: on a timeout the kernel records
// kStatusPeerTimeout and returns.  The signalling store is a plain st.release.sys after cp.async.bulk.wait_group 0:
// an extra __threadfence_system() in front of it cost 10-25 us per tile while TMA loads were in flight.
//
// Reduce-scatter form (GemmArComm::scatter): the owner of a tile is the rank that keeps its ROWS, the owner warps
// write the reduced rows to the local [M / tp][N] output and push nothing, the receiver warps have no work.  Used for
// the backward of an all-gather -> GEMM (the gradient of the gathered input is needed only on the rank the rows came
// from): half the NVLink bytes of the all-reduce form.
#include <cuda.h>

#include "common.cuh"
#include "gemm_ar_sm100.cuh"
#include "gemm_sm100.cuh"

namespace ssb {

int make_tma_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                     uint32_t box_rows, uint32_t box_cols);


namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kThreads = 64 + 128 + 128 + 128;  // TMA, MMA | partial epilogue | owner role | receiver role
constexpr int kABytes = BM * BK * 2, kBBytes = BN * BK * 2, kStageBytes = kABytes + kBBytes;
constexpr int kChunkBytes = 32 * 32 * 2;            // one 32-row x 32-column bf16 piece of a partial tile
constexpr int kStageEBytes = 4 * 2 * kChunkBytes;  // partial-epilogue staging: 4 warps x 2 buffers
constexpr int kStageCBytes = 4 * 8 * BN * 2;        // collective staging: 4 warps x 8 rows x 512 B
constexpr int kSmemBytes = kStages * kStageBytes + kStageEBytes + kStageCBytes + 1024 + 256;
constexpr int kGroupM = 8;
constexpr int kTileElems = BM * BN;
constexpr uint64_t kPeerLimitNs = 20ull * 1000 * 1000 * 1000;

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait until *flag >= epoch.  Warp-uniform result.
__device__ __forceinline__ bool wait_flag_warp(const uint32_t* flag, bool active, uint32_t epoch, volatile int* abort_flag,
                                               int* status) {
  bool ok = true;
  if (active) {
    ok = false;
    uint64_t t0 = 0;
    for (uint32_t it = 0; it < (1u << 30); ++it) {
      if (ld_acquire_sys_u32(flag) >= epoch) { ok = true; break; }
      if ((it & 1023u) == 1023u) {
        if (*abort_flag) break;
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > kPeerLimitNs) break;
      }
    }
    if (!ok) {
      *abort_flag = 1;
      if (status != nullptr) atomicMax(status, static_cast<int>(kStatusPeerTimeout));
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  __syncwarp();  // orders the other lanes' data reads after the polling lanes' acquire
  return ok;
}
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Asynchronous copy shared memory -> global memory (this GPU's or a peer's), tracked by the bulk async-group of the
// issuing thread.  Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_copy_s2g(void* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes)
               : "memory");
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

// Final epilogue on 8 consecutive columns [n0, n0+8) of row `row`: bias, dropout, residual (see GemmParams).
// `row` is the row of the full [M][N] product (it enters the dropout counter, so the mask does not depend on how
// the rows are dealt out), `mem_row` the row of p.residual that holds it (differs in the reduce-scatter form).
__device__ __forceinline__ uint4 final_epilogue8(const GemmParams& p, int row, int mem_row, int n0, float (&v)[8],
                                                 uint32_t keep16, float drop_scale) {
  if (p.bias != nullptr) {
    if (p.bias_fp32) {
      const float4 b0 = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.bias) + n0));
      const float4 b1 = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.bias) + n0) + 1);
      v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
      v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
    } else {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.bias) + n0));
      float2 f;
      f = unpack_bf16x2(q.x); v[0] += f.x; v[1] += f.y;
      f = unpack_bf16x2(q.y); v[2] += f.x; v[3] += f.y;
      f = unpack_bf16x2(q.z); v[4] += f.x; v[5] += f.y;
      f = unpack_bf16x2(q.w); v[6] += f.x; v[7] += f.y;
    }
  }
  if (p.dropout_p > 0.f) {
    const uint64_t g0 = (static_cast<uint64_t>(row) * static_cast<uint64_t>(p.N) + n0) >> 2;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const uint32_t m = dropout_keep4(p.dropout_seed, g0 + g, keep16);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[4 * g + i] = ((m >> i) & 1u) ? v[4 * g + i] * drop_scale : 0.f;
    }
  }
  if (p.residual != nullptr) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.residual) +
                                                         static_cast<size_t>(mem_row) * p.ldres + n0));
    float2 f;
    f = unpack_bf16x2(q.x); v[0] += f.x; v[1] += f.y;
    f = unpack_bf16x2(q.y); v[2] += f.x; v[3] += f.y;
    f = unpack_bf16x2(q.z); v[4] += f.x; v[5] += f.y;
    f = unpack_bf16x2(q.w); v[6] += f.x; v[7] += f.y;
  }
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]);
  o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]);
  o.w = pack_bf16x2(v[6], v[7]);
  return o;
}

template <bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_ar_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const GemmParams p, const GemmArComm cm) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kABytes;
  uint8_t* stage_e = smem + kStages * kStageBytes;
  uint8_t* stage_c = stage_e + kStageEBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_c + kStageCBytes);
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
  // flag table of a rank: [max_tiles][tp][4] "partial quarter written", then [max_tiles][4] "quarter final"
  const int part_flags_per_tile = cm.tp * 4;
  const size_t final_base = static_cast<size_t>(cm.max_tiles) * part_flags_per_tile;
  const int slots = (num_tiles + cm.tp - 1) / cm.tp;  // tiles owned by one rank
  // Owner of a tile: inside every group of tp consecutive tiles the owners are a rotation of 0..tp-1 (so slot =
  // tile / tp is unique per owner), and the rotation advances once per sweep of the grid, so a CTA alternates
  // between owned and foreign tiles instead of owning all of its tiles.
  const int rot_div = max(1, cm.grid / cm.tp);
  // reduce-scatter form: the owner is the rank that keeps the tile's rows; its slot is the tile's index among them
  const int mb_per_rank = cm.scatter ? (p.M / cm.tp) / BM : 1;
  auto owner_of = [&](int tile) {
    if (cm.scatter) return tile_coord(tile, num_m, num_n).m_blk / mb_per_rank;
    return (tile % cm.tp + (tile / cm.tp) / rot_div) % cm.tp;
  };
  auto slot_of = [&](int tile) {
    if (cm.scatter) {
      const TileCoord c = tile_coord(tile, num_m, num_n);
      return (c.m_blk % mb_per_rank) * num_n + c.n_blk;
    }
    return tile / cm.tp;
  };
  uint32_t* const consumed_flags_mine = cm.flag_ptrs[cm.rank] + final_base + static_cast<size_t>(cm.max_tiles) * 4;

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
    tmem_alloc(tmem_slot, 2 * BN);
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
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, num_m, num_n);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
          uint8_t* sa = smem_a + stage * kABytes;
          uint8_t* sb = smem_b + stage * kBBytes;
          tma_load_2d(sa, &tma_a, &full_bar[stage], kb * BK, tc.m_blk * BM);
          if (!B_MN) {
            tma_load_2d(sb, &tma_b, &full_bar[stage], kb * BK, tc.n_blk * BN);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (64 * BK * 2), &tma_b, &full_bar[stage], tc.n_blk * BN + c * 64, kb * BK);
          }
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
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, false, B_MN);
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
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = umma_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_desc_sw128(sb + k * 2048, 64 * BK * 2, 1024)
                                     : umma_desc_sw128(sb + k * 32, 16, 1024);
            umma_f16_ss(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full_bar[acc]);
      }
    }
  } else if (warp < 6) {
    // ---------- partial epilogue: TMEM -> bf16 -> staging in shared memory -> bulk copy into the owner's scratch ----------
    const int quarter = warp & 3;
    uint8_t* stage = stage_e + (warp - 2) * (2 * kChunkBytes);  // two 2 KB buffers per warp
    int iter = 0;
    bool ok = true;
    // every owner has finished reading what the last reduce-scatter call left in its scratch
    if (cm.wait_consumed_epoch != 0)
      ok = wait_flag_warp(consumed_flags_mine + lane, lane < cm.tp, cm.wait_consumed_epoch, abort_flag, p.status);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++iter) {
      const int acc = iter & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full_bar[acc], (iter >> 1) & 1, abort_flag))) { ok = false; break; }
      tc_fence_after_sync();
      const int owner = owner_of(tile);
      // slot of this (source rank, tile) in the owner's scratch; inside a slot: [quarter][32-column chunk][32 rows][64 B]
      uint8_t* dst = reinterpret_cast<uint8_t*>(const_cast<void*>(cm.partial_ptrs[owner])) +
                     ((static_cast<size_t>(cm.rank) * slots + slot_of(tile)) * kTileElems) * 2 +
                     static_cast<size_t>(quarter) * (32 * BN * 2);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (c == BN / 32 - 1) {  // the accumulator stage is free as soon as its last columns are in registers
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
        }
        uint8_t* buf = stage + (c & 1) * kChunkBytes;
        if (lane == 0) tma_store_wait_read<1>();  // the copy that last read this buffer has fetched it
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 q;
          q.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]) * p.alpha, __uint_as_float(r[8 * i + 1]) * p.alpha);
          q.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * p.alpha, __uint_as_float(r[8 * i + 3]) * p.alpha);
          q.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * p.alpha, __uint_as_float(r[8 * i + 5]) * p.alpha);
          q.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * p.alpha, __uint_as_float(r[8 * i + 7]) * p.alpha);
          *reinterpret_cast<uint4*>(buf + lane * 64 + i * 16) = q;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          bulk_copy_s2g(dst + c * kChunkBytes, buf, kChunkBytes);
          tma_store_commit();
        }
      }
      if (lane == 0) {
        tma_store_wait<0>();       // every chunk of this quarter has been written to the owner's memory
        st_release_sys_u32(cm.flag_ptrs[owner] + static_cast<size_t>(tile) * part_flags_per_tile + cm.rank * 4 + quarter,
                           cm.epoch);
      }
      __syncwarp();
    }
  } else {
    // ----------------------------- collective warps -----------------------------
    const int quarter = warp & 3;  // warps 6..9 -> quarters 2,3,0,1: any bijection works
    const uint32_t keep16 = dropout_keep16(p.dropout_p);
    const float drop_scale = p.dropout_p > 0.f ? 65536.0f / static_cast<float>(keep16) : 1.0f;
    uint32_t* my_flags = cm.flag_ptrs[cm.rank];
    const __nv_bfloat16* my_partial = reinterpret_cast<const __nv_bfloat16*>(cm.partial_ptrs[cm.rank]);
    const __nv_bfloat16* my_result = reinterpret_cast<const __nv_bfloat16*>(cm.result_ptrs[cm.rank]);
    constexpr int R = 8;  // rows per batch
    const bool owner_role = warp < 10;  // warps 6..9 reduce and publish owned tiles, warps 10..13 receive foreign ones
    uint8_t* stage = stage_c + (quarter) * (R * BN * 2);  // 4 KB per owner-role warp
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const TileCoord tc = tile_coord(tile, num_m, num_n);
      const int owner = owner_of(tile);
      const int row0 = tc.m_blk * BM + quarter * 32;
      const int col = tc.n_blk * BN + lane * 8;  // this lane's 8 columns of every row
      const bool col_ok = col < p.N;             // N is a multiple of 8
      const int rows = min(32, p.M - row0);      // may be <= 0 on the ragged edge
      if ((owner == cm.rank) != owner_role) continue;
      if (cm.scatter && !owner_role) continue;  // reduce-scatter: nothing comes back
      const int mem_row0 = cm.scatter ? row0 - cm.rank * (p.M / cm.tp) : row0;  // row of the local output
      if (owner_role) {
        ok = wait_flag_warp(my_flags + static_cast<size_t>(tile) * part_flags_per_tile + lane * 4 + quarter,
                            lane < cm.tp, cm.epoch, abort_flag, p.status);
        if (!ok) break;
        // partial slots are stored [quarter][chunk][row][64 B]: this lane's 8 columns sit in chunk lane / 4
        const size_t slot_off = static_cast<size_t>(slot_of(tile)) * kTileElems + static_cast<size_t>(quarter) * (32 * BN) +
                                (lane >> 2) * (32 * 32) + (lane & 3) * 8;
        const size_t res_off = static_cast<size_t>(tile) * kTileElems + static_cast<size_t>(quarter) * (32 * BN);
#pragma unroll 1
        for (int rb = 0; rb < 32; rb += R) {
          if (rb >= rows) break;
          float v[R][8];
#pragma unroll
          for (int i = 0; i < R; ++i)
#pragma unroll
            for (int e = 0; e < 8; ++e) v[i][e] = 0.f;
          for (int r = 0; r < cm.tp; ++r) {
            const __nv_bfloat16* src = my_partial + static_cast<size_t>(r) * slots * kTileElems + slot_off;
            uint4 q[R];
#pragma unroll
            for (int i = 0; i < R; ++i) q[i] = ld_nc_v4(src + (rb + i) * 32);
#pragma unroll
            for (int i = 0; i < R; ++i) {
              float2 f;
              f = unpack_bf16x2(q[i].x); v[i][0] += f.x; v[i][1] += f.y;
              f = unpack_bf16x2(q[i].y); v[i][2] += f.x; v[i][3] += f.y;
              f = unpack_bf16x2(q[i].z); v[i][4] += f.x; v[i][5] += f.y;
              f = unpack_bf16x2(q[i].w); v[i][6] += f.x; v[i][7] += f.y;
            }
          }
          if (cm.scatter) {
#pragma unroll
            for (int i = 0; i < R; ++i) {
              if (col_ok && rb + i < rows) {
                const uint4 o = final_epilogue8(p, row0 + rb + i, mem_row0 + rb + i, col, v[i], keep16, drop_scale);
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.D) +
                                          static_cast<size_t>(mem_row0 + rb + i) * p.ldd + col) = o;
              }
            }
            continue;
          }
          if (lane == 0) tma_store_wait_read<0>();  // the previous batch has left the staging buffer
          __syncwarp();
#pragma unroll
          for (int i = 0; i < R; ++i) {
            const int row = row0 + rb + i;
            uint4 o = make_uint4(0u, 0u, 0u, 0u);
            if (col_ok && rb + i < rows) {
              o = final_epilogue8(p, row, row, col, v[i], keep16, drop_scale);
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<size_t>(row) * p.ldd + col) = o;
            }
            *reinterpret_cast<uint4*>(stage + i * (BN * 2) + lane * 16) = o;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            // push the batch (8 rows x 512 B, contiguous in the row-major result tile) to every peer
            for (int pr = 0; pr < cm.tp; ++pr)
              if (pr != cm.rank)
                bulk_copy_s2g(reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(cm.result_ptrs[pr])) + res_off +
                                  static_cast<size_t>(rb) * BN,
                              stage, R * BN * 2);
            tma_store_commit();
          }
        }
        if (lane == 0 && !cm.scatter) {
          tma_store_wait<0>();
          for (int pr = 0; pr < cm.tp; ++pr)
            if (pr != cm.rank)
              st_release_sys_u32(cm.flag_ptrs[pr] + final_base + static_cast<size_t>(tile) * 4 + quarter, cm.epoch);
        }
        __syncwarp();
      } else {
        ok = wait_flag_warp(my_flags + final_base + static_cast<size_t>(tile) * 4 + quarter, lane == 0, cm.epoch,
                            abort_flag, p.status);
        if (!ok) break;
        const __nv_bfloat16* src = my_result + static_cast<size_t>(tile) * kTileElems +
                                   static_cast<size_t>(quarter * 32) * BN + lane * 8;
#pragma unroll 1
        for (int rb = 0; rb < 32; rb += R) {
          if (rb >= rows) break;
          uint4 q[R];
#pragma unroll
          for (int i = 0; i < R; ++i) q[i] = ld_nc_v4(src + static_cast<size_t>(rb + i) * BN);
#pragma unroll
          for (int i = 0; i < R; ++i)
            if (col_ok && rb + i < rows)
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.D) +
                                        static_cast<size_t>(row0 + rb + i) * p.ldd + col) = q[i];
        }
      }
    }
    if (lane == 0) tma_store_wait<0>();
    if (cm.scatter && owner_role && ok) {
      // Publish "consumed": the four owner warps of every CTA count themselves; the last one of the grid resets the
      // counter for the next call and tells every peer that this rank has read all the partials of this epoch.
      __syncwarp();
      if (lane == 0) {
        uint32_t* counter = consumed_flags_mine + cm.tp;
        __threadfence();
        const uint32_t seen = atomicAdd(counter, 1u);
        if (seen == 4u * gridDim.x - 1u) {
          *counter = 0u;
          __threadfence_system();
          for (int pr = 0; pr < cm.tp; ++pr)
            st_release_sys_u32(cm.flag_ptrs[pr] + final_base + static_cast<size_t>(cm.max_tiles) * 4 + cm.rank, cm.epoch);
        }
      }
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


// A [M][K] bf16 (K contiguous); B [N][K] (b_mn_major = 0) or [K][N] (1).  p describes the FINAL epilogue
// (alpha, bias, dropout, residual) and the local bf16 output; activation / pre-activation / accumulate / fp32
// outputs are not available in the fused form.  N must be a multiple of 32.
int gemm_ar_launch(const void* A, int lda, const void* B, int ldb, int b_mn_major, const GemmParams& p,
                   const GemmArComm& cm, int num_sms, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0 || p.K <= 0 || (p.N % 32)) return -2;
  if (p.act != kActNone || p.preact_out != nullptr || p.accumulate || p.out_fp32) return -2;
  if ((lda % 8) || (ldb % 8) || (p.ldd % 8)) return -3;
  const int num_tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  if (num_tiles > cm.max_tiles || cm.tp < 1 || cm.tp > 32) return -6;
  if (cm.scatter && (p.M % (cm.tp * BM))) return -2;  // every rank keeps whole 128-row blocks
  if (static_cast<long long>(num_tiles + cm.tp) * kTileElems > cm.capacity_elems) return -6;
  CUtensorMap ta, tb;
  int rc = make_tma_2d_bf16(&ta, A, p.M, p.K, lda, BM, BK);
  if (rc != 0) return rc;
  rc = !b_mn_major ? make_tma_2d_bf16(&tb, B, p.N, p.K, ldb, BN, BK) : make_tma_2d_bf16(&tb, B, p.K, p.N, ldb, BK, 64);
  if (rc != 0) return rc;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_ar_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_ar_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done = true;
  }
  const int grid = num_tiles < num_sms ? num_tiles : num_sms;
  GemmArComm c2 = cm;
  c2.grid = grid;  // the same on every rank: it enters the tile -> owner map
  if (b_mn_major)
    gemm_ar_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, p, c2);
  else
    gemm_ar_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, p, c2);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ssb
