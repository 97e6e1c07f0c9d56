// Two-SM ("cta_group::2") variant of the bf16 GEMM: a cluster of two CTAs on one SM pair computes a
// 256 x 256 output tile.  Each CTA stages its own 128 rows of A and its own 128 of the tile's 256 B rows
// (columns of the output), the leader CTA issues tcgen05.mma.cta_group::2 instructions that read both
// CTAs' shared memory, and each CTA ends up with its 128 x 256 half of the accumulator in its own TMEM.
//
// Why: with one CTA per 128 x 256 tile the tensor core reads 12 KB of operands from shared memory per
// 128 x 256 x 16 step while TMA writes the same amount, which exceeds what one SM's shared memory delivers
// (measured: tensor pipe 65 % busy, L1/shared pipe 80 %).  Pairing halves the B traffic per SM.
//
//   warp 0     : TMA producer (one elected lane), in both CTAs
//   warp 1     : TMEM allocator in both CTAs; MMA issuer in the leader (cluster rank 0)
//   warps 2..17: epilogue; warp w reads TMEM lanes 32*(w%4)..+31, columns 64*((w-2)/4)..+63 in chunks of 16.
//                Sixteen warps (four per SM sub-partition): with eight, bias + GeLU + pre-activation epilogues took
//                longer than the K = 2048 main loop of the next tile (measured 643 us against 407 us for the same
//                GEMM with a plain epilogue)
//
// Barriers: `full` lives in the leader and counts the bytes of both CTAs' loads (the peer's TMA signals it
// through the cluster address); `empty` and `tmem_full` exist in both CTAs and are signalled together by a
// multicast tcgen05.commit; `tmem_empty` lives in the leader and collects the epilogue warps of both CTAs.
// Same operation and epilogue as gemm_bf16_kernel (runtime/megatron/mpu/layers.py:363,459,532,593 of the
// reference are the call sites this replaces).
#include <cuda.h>

#include "common.cuh"
#include "gemm_ag_sm100.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_sm100.cuh"

namespace ssb {

int make_tma_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                     uint32_t box_rows, uint32_t box_cols);

namespace {

constexpr int BM2 = 128;   // rows per CTA (256 per cluster)
constexpr int BNH = 128;   // B rows staged per CTA (256 output columns per cluster)
constexpr int BN2 = 256;
constexpr int BK2 = 64;
constexpr int kStagesPlain = 5;
constexpr int kStagesGather = 4;                 // one stage (32 KB) becomes the pusher's staging area
constexpr int kPushChunk2 = 16384;
constexpr int kEpiWarps = 16;
constexpr int kThreads2 = 64 + kEpiWarps * 32;
constexpr int kThreadsGather = kThreads2 + 32;    // + pusher warp
constexpr int kGroupM2 = 8;
constexpr int kABytes2 = BM2 * BK2 * 2;
constexpr int kBBytes2 = BNH * BK2 * 2;
constexpr int kStageBytes2 = kABytes2 + kBBytes2;
constexpr int kEpiStage = 32 * 128;                 // per epilogue warp: 32 rows x 64 bf16 columns, 128-byte swizzle
constexpr int kSmem2 = kStagesPlain * kStageBytes2 + kEpiWarps * kEpiStage + 1024 + 256;  // both variants

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_smem(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory whose completion bytes are counted on an mbarrier that may live in
// the other CTA of the pair (no multicast: every CTA fetches its own tile).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this offset in BOTH CTAs once all MMAs issued so far have retired.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}

// TMEM allocation for a CTA pair: warp 1 of BOTH CTAs executes these, with the same shared-memory offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Bounded wait (one thread) until *flag >= epoch.
__device__ __forceinline__ bool wait_flag_one(const uint32_t* flag, uint32_t epoch, volatile int* abort_flag, int* status) {
  uint64_t t0 = 0;
  for (uint32_t it = 0; it < (1u << 30); ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= epoch) return true;
    if ((it & 1023u) == 1023u) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 20ull * 1000 * 1000 * 1000) break;
    }
  }
  *abort_flag = 1;
  if (status != nullptr) atomicMax(status, static_cast<int>(kStatusPeerTimeout));
  return false;
}

struct TileCoord2 {
  int m_blk, n_blk;
};
__device__ __forceinline__ TileCoord2 tile_coord2(int tile, int num_m, int num_n) {
  const int per_group = kGroupM2 * num_n;
  const int group = tile / per_group;
  const int first_m = group * kGroupM2;
  const int gsize = min(num_m - first_m, kGroupM2);
  const int in_group = tile - group * per_group;
  TileCoord2 c;
  c.m_blk = first_m + in_group % gsize;
  c.n_blk = in_group / gsize;
  return c;
}

// GATHER = true: the all-gather of A's rows over the tensor-parallel group is part of the kernel (see
// gemm_ag_sm100.cu for the protocol): tma_a addresses this rank's own rows, tma_a2 the local gather buffer, output
// tiles are ordered own rows first, the producer waits for the "arrived" flag of a 128-row block before loading it,
// and warp 18 pushes this rank's rows to every peer.
template <bool A_MN, bool B_MN, bool GATHER>
__global__ void __launch_bounds__(GATHER ? kThreadsGather : kThreads2, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_a2,
                  const __grid_constant__ CUtensorMap tma_b, const GemmParams p, const GemmAgComm cm) {
  constexpr int kStages2 = GATHER ? kStagesGather : kStagesPlain;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages2 * kABytes2;
  uint8_t* push_buf = smem + kStages2 * kStageBytes2;              // GATHER only: 2 x 16 KB
  uint8_t* epi_stage = push_buf + (GATHER ? 2 * kPushChunk2 : 0);
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + kEpiWarps * kEpiStage);
  uint64_t* full_bar = bars;                       // leader's are used
  uint64_t* empty_bar = bars + kStages2;           // both CTAs
  uint64_t* tmem_full_bar = bars + 2 * kStages2;   // both CTAs
  uint64_t* tmem_empty_bar = bars + 2 * kStages2 + 2;  // leader's are used
  uint64_t* push_bar = bars + 2 * kStages2 + 4;  // 2 (GATHER only)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages2 + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  const int num_m = (p.M + 2 * BM2 - 1) / (2 * BM2);
  const int num_n = (p.N + BN2 - 1) / BN2;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK2 - 1) / BK2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tmem_full_bar[s], 1);
      mbar_init(&tmem_empty_bar[s], 2 * kEpiWarps);
      mbar_init(&push_bar[s], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // GATHER: logical pair-block i (the order tiles are computed in) -> source rank and actual pair-block
  const int pb_per_rank = GATHER ? max(1, num_m / cm.tp) : 1;
  auto src_of = [&](int i) { return GATHER ? (cm.rank + i / pb_per_rank) % cm.tp : 0; };
  auto pblk_of = [&](int i) { return GATHER ? src_of(i) * pb_per_rank + i % pb_per_rank : i; };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const TileCoord2 tc = tile_coord2(tile, num_m, num_n);
        int m0 = pblk_of(tc.m_blk) * 2 * BM2 + static_cast<int>(cta_rank) * BM2;
        const int n0 = tc.n_blk * BN2 + static_cast<int>(cta_rank) * BNH;
        const CUtensorMap* ta = &tma_a;
        if (GATHER) {
          if (src_of(tc.m_blk) == cm.rank) {
            m0 -= cm.rank * pb_per_rank * 2 * BM2;  // own rows: read straight from the local shard
          } else {
            // rows pushed by another rank: wait for this CTA's 128-row block, then order the TMA reads after it
            if (!wait_flag_one(cm.flag_ptrs[cm.rank] + m0 / BM2, cm.epoch, abort_flag, p.status)) { ok = false; break; }
            asm volatile("fence.proxy.async.global;" ::: "memory");
            ta = &tma_a2;
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * kStageBytes2);
          const uint32_t bar = mapa_smem(smem_u32(&full_bar[stage]), 0);
          uint8_t* sa = smem_a + stage * kABytes2;
          uint8_t* sb = smem_b + stage * kBBytes2;
          if (!A_MN) {
            tma_load_2d_pair(sa, ta, bar, kb * BK2, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM2 / 64; ++c) tma_load_2d_pair(sa + c * (64 * BK2 * 2), ta, bar, m0 + c * 64, kb * BK2);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tma_b, bar, kb * BK2, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BNH / 64; ++c) tma_load_2d_pair(sb + c * (64 * BK2 * 2), &tma_b, bar, n0 + c * 64, kb * BK2);
          }
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      // The copies issued by this thread have landed once the MMAs that consume them retired, which the
      // epilogue of the last tile waits for; on an aborted run the teardown below waits for them instead.
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (leader && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM2, BN2, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN2;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem_a + stage * kABytes2);
          const uint32_t sb = smem_u32(smem_b + stage * kBBytes2);
#pragma unroll
          for (int k = 0; k < BK2 / 16; ++k) {
            const uint64_t da = A_MN ? umma_desc_sw128(sa + k * 2048, 64 * BK2 * 2, 1024)
                                     : umma_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_desc_sw128(sb + k * 2048, 64 * BK2 * 2, 1024)
                                     : umma_desc_sw128(sb + k * 32, 16, 1024);
            umma_f16_ss_pair(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage]);
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit_pair(&tmem_full_bar[acc]);
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // -------------------------------- epilogue --------------------------------
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;  // 64-column group of the 256-column tile
    uint8_t* stg = epi_stage + (warp - 2) * kEpiStage;
    const uint32_t keep16 = dropout_keep16(p.dropout_p);
    const float drop_scale = p.dropout_p > 0.f ? 65536.0f / static_cast<float>(keep16) : 1.0f;
    int iter = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++iter) {
      const TileCoord2 tc = tile_coord2(tile, num_m, num_n);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      const int row0 = pblk_of(tc.m_blk) * 2 * BM2 + static_cast<int>(cta_rank) * BM2 + quarter * 32;  // first row of this warp
      const int col0 = tc.n_blk * BN2 + grp * 64;                                              // first column
      const int row = row0 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN2 + grp * 64;
      // Staged path: bf16 output, no accumulate, the warp's 64 columns inside the matrix, at most one row operand.
      // Row operands enter and results leave through a 4 KB swizzled staging tile, so every global access of the
      // warp is four full 128-byte row segments instead of 32 scattered 32-byte pieces.
      const bool has_operand = p.residual != nullptr || p.act == kActDGelu || p.act == kActDRelu;
      const bool staged = !p.out_fp32 && !p.accumulate && col0 + 64 <= p.N &&
                          !(p.residual != nullptr && (p.act == kActDGelu || p.act == kActDRelu)) &&
                          !(p.preact_out != nullptr && has_operand);
      if (staged) {
        const int srow = lane >> 3, spiece = lane & 7;  // coalesced phase: 4 rows x 8 sixteen-byte pieces per pass
        auto cell = [&](int rr, int piece) { return stg + rr * 128 + ((piece ^ (rr & 7)) << 4); };
        if (has_operand) {  // fetched while the tensor cores still work on this tile
          const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(p.residual != nullptr ? p.residual : p.aux);
          const int ld = p.residual != nullptr ? p.ldres : p.ldaux;
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + srow;
            if (row0 + rr < p.M)
              *reinterpret_cast<uint4*>(cell(rr, spiece)) =
                  __ldg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(row0 + rr) * ld + col0) + spiece);
          }
          __syncwarp();
        }
        if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        auto flush = [&](void* base, int ld) {  // staging tile -> global, 4 rows x 128 bytes per instruction
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + srow;
            if (row0 + rr < p.M)
              *(reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + static_cast<size_t>(row0 + rr) * ld + col0) +
                spiece) = *reinterpret_cast<const uint4*>(cell(rr, spiece));
          }
          __syncwarp();
        };
        if (p.preact_out != nullptr) {  // first pass: the pre-activation tile
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[16];
            tmem_ld_32x16(taddr + c * 16, r);
            tmem_ld_wait();
            const uint4 none[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
            float pre[16], v[16];
            gemm_epilogue_math16(p, row, col0 + c * 16, r, none, keep16, drop_scale, pre, v);
            *reinterpret_cast<uint4*>(cell(lane, 2 * c)) = pack8(pre);
            *reinterpret_cast<uint4*>(cell(lane, 2 * c + 1)) = pack8(pre + 8);
          }
          flush(p.preact_out, p.ldpre);
        }
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[16];
          tmem_ld_32x16(taddr + c * 16, r);
          tmem_ld_wait();
          if (c == 3) {  // the accumulator stage is free once its last columns are in registers
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_smem(smem_u32(&tmem_empty_bar[acc]), 0));
          }
          uint4 operand[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
          if (has_operand) {
            operand[0] = *reinterpret_cast<const uint4*>(cell(lane, 2 * c));
            operand[1] = *reinterpret_cast<const uint4*>(cell(lane, 2 * c + 1));
          }
          float pre[16], v[16];
          gemm_epilogue_math16(p, row, col0 + c * 16, r, operand, keep16, drop_scale, pre, v);
          *reinterpret_cast<uint4*>(cell(lane, 2 * c)) = pack8(v);
          *reinterpret_cast<uint4*>(cell(lane, 2 * c + 1)) = pack8(v + 8);
        }
        flush(p.D, p.ldd);
        continue;
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag))) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        const int n0 = col0 + c * 16;
        if (n0 >= p.N) break;  // uniform across the warp
        uint32_t r[16];
        tmem_ld_32x16(taddr + c * 16, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        gemm_epilogue_chunk<16>(p, row, n0, r, keep16, drop_scale);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_smem(smem_u32(&tmem_empty_bar[acc]), 0));
    }
  } else if (GATHER) {
    // --------------------------------- pusher ---------------------------------
    // Copies this rank's rows, 128-row block by block (CTA c takes blocks c, c + grid, ...), through a double-
    // buffered 16 KB staging area into the same rows of every peer's gather buffer, then flags the block there.
    if (lane == 0 && cm.tp > 1) {
      const size_t blk_bytes = static_cast<size_t>(BM2) * p.K * 2;  // shard and gather buffers are dense
      const uint8_t* x = reinterpret_cast<const uint8_t*>(cm.x_local);
      const int blocks_per_rank = pb_per_rank * 2;
      const int pieces_per_blk = static_cast<int>(blk_bytes / kPushChunk2);
      int my_blocks = 0;
      for (int b = blockIdx.x; b < blocks_per_rank; b += gridDim.x) ++my_blocks;
      const int total = my_blocks * pieces_per_blk;
      auto issue_load = [&](int j) {
        const int b = blockIdx.x + (j / pieces_per_blk) * gridDim.x;
        mbar_arrive_expect_tx(&push_bar[j & 1], kPushChunk2);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         smem_u32(push_buf + (j & 1) * kPushChunk2)),
                     "l"(x + static_cast<size_t>(b) * blk_bytes + static_cast<size_t>(j % pieces_per_blk) * kPushChunk2),
                     "r"(kPushChunk2), "r"(smem_u32(&push_bar[j & 1]))
                     : "memory");
      };
      bool okp = true;
      if (total > 0) issue_load(0);
      for (int j = 0; j < total && okp; ++j) {
        if (j + 1 < total) {
          tma_store_wait_read<0>();  // the stores of piece j - 1 have left the other buffer
          issue_load(j + 1);
        }
        if (!mbar_wait(&push_bar[j & 1], (j >> 1) & 1, abort_flag)) { okp = false; break; }
        const int b = blockIdx.x + (j / pieces_per_blk) * gridDim.x;
        const size_t dst_off = (static_cast<size_t>(cm.rank) * blocks_per_rank + b) * blk_bytes +
                               static_cast<size_t>(j % pieces_per_blk) * kPushChunk2;
        for (int pr = 0; pr < cm.tp; ++pr)
          if (pr != cm.rank)
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                             reinterpret_cast<uint8_t*>(cm.gather_ptrs[pr]) + dst_off),
                         "r"(smem_u32(push_buf + (j & 1) * kPushChunk2)), "r"(kPushChunk2)
                         : "memory");
        tma_store_commit();
        if (j % pieces_per_blk == pieces_per_blk - 1) {
          tma_store_wait<0>();  // the whole block has been written on every peer
          for (int pr = 0; pr < cm.tp; ++pr)
            if (pr != cm.rank)
              asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(cm.flag_ptrs[pr] + cm.rank * blocks_per_rank + b),
                           "r"(cm.epoch)
                           : "memory");
        }
      }
      tma_store_wait<0>();
    }
  }

  // ------------------------------- teardown ----------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // Aborted: give the copies in flight into this CTA's shared memory a bounded time to land.
    if (threadIdx.x == 0) {
      if (p.status != nullptr) atomicMax(p.status, static_cast<int>(kStatusMbarTimeout));
      const uint64_t t0 = global_timer_ns();
      for (uint32_t it = 0; it < (1u << 22); ++it)
        if (global_timer_ns() - t0 > 2000000ull) break;
    }
    __syncthreads();
  }
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while the other may still address it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <bool A_MN, bool B_MN, bool GATHER>
int launch_pair(const void* A, int lda, const void* B, int ldb, const GemmParams& p, const GemmAgComm& cm, int num_sms,
                cudaStream_t stream) {
  CUtensorMap ta, ta2, tb;
  int rc;
  if (GATHER) {  // A = this rank's rows [M / tp][K]; the gather buffer holds all M rows
    rc = make_tma_2d_bf16(&ta, A, p.M / cm.tp, p.K, lda, BM2, BK2);
    if (rc != 0) return rc;
    rc = make_tma_2d_bf16(&ta2, cm.gather_ptrs_host_local, p.M, p.K, p.K, BM2, BK2);
  } else {
    rc = !A_MN ? make_tma_2d_bf16(&ta, A, p.M, p.K, lda, BM2, BK2) : make_tma_2d_bf16(&ta, A, p.K, p.M, lda, BK2, 64);
    ta2 = ta;
  }
  if (rc != 0) return rc;
  rc = !B_MN ? make_tma_2d_bf16(&tb, B, p.N, p.K, ldb, BNH, BK2) : make_tma_2d_bf16(&tb, B, p.K, p.N, ldb, BK2, 64);
  if (rc != 0) return rc;
  auto kernel = gemm2_bf16_kernel<A_MN, B_MN, GATHER>;
  constexpr int threads = GATHER ? kThreadsGather : kThreads2;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  static int max_clusters = 0;
  if (max_clusters == 0) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(num_sms & ~1);
    q.blockDim = dim3(threads);
    q.dynamicSmemBytes = kSmem2;
    q.attrs = attr;
    q.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kernel, &q);
    if (e != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      return -5;
    }
    max_clusters = n;
  }
  const int num_tiles = ((p.M + 2 * BM2 - 1) / (2 * BM2)) * ((p.N + BN2 - 1) / BN2);
  int clusters = num_sms / 2;
  if (clusters > max_clusters) clusters = max_clusters;
  if (clusters > num_tiles) clusters = num_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = kSmem2;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, ta, ta2, tb, p, cm));
}

}  // namespace

// Same contract as gemm_bf16_launch; callers pick this variant for outputs of at least 256 x 256.
int gemm2_bf16_launch(const void* A, int lda, int a_mn_major, const void* B, int ldb, int b_mn_major,
                      const GemmParams& p, int num_sms, cudaStream_t stream) {
  const GemmAgComm none{};
  if (!a_mn_major && !b_mn_major) return launch_pair<false, false, false>(A, lda, B, ldb, p, none, num_sms, stream);
  if (!a_mn_major && b_mn_major) return launch_pair<false, true, false>(A, lda, B, ldb, p, none, num_sms, stream);
  if (a_mn_major && b_mn_major) return launch_pair<true, true, false>(A, lda, B, ldb, p, none, num_sms, stream);
  return launch_pair<true, false, false>(A, lda, B, ldb, p, none, num_sms, stream);
}

// All-gather fused into the GEMM on the two-SM kernel.  Returns -100 when the shape does not fit this variant
// (rows per rank not a multiple of 256, narrow output): the caller then uses the one-CTA kernel of gemm_ag_sm100.cu.
int gemm2_ag_launch(const void* W, int ldw, const GemmParams& p, const GemmAgComm& cm, int num_sms, cudaStream_t stream) {
  const int rows_local = p.M / cm.tp;
  if (rows_local % (2 * BM2) || p.N < BN2 || (static_cast<size_t>(BM2) * p.K * 2) % kPushChunk2) return -100;
  return launch_pair<false, false, true>(cm.x_local, p.K, W, ldw, p, cm, num_sms, stream);
}

}  // namespace ssb
