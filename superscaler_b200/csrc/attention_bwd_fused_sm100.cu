// Flash-attention backward in ONE kernel for sm_100a: five tile GEMMs per (key block, query block) pair on tcgen05
// tensor cores instead of the seven of the dK/dV + dQ kernel pair, and one pass of the exponentials, the dropout mask
// and the dS arithmetic instead of two.
//
// Replaces the autograd of ParallelAttentionScoreOp / SoftmaxFusion / SoftmaxDropout / ContextOp
// (runtime/megatron/model/flex_ops.py:711-1015) together with the softmax backward kernels of the reference
// (runtime/megatron/fused_kernels/scaled_masked_softmax.h:329-423).
//
// A CTA owns 128 keys of one (batch, head) and walks over the query blocks (64 queries each) that see them:
//   S^T  = K . Q_i^T          [128 keys x 64 queries]     TMEM columns [0, 64)
//   dP^T = V . dO_i^T         [128 keys x 64 queries]     TMEM columns [64, 128)
//   math : P^T = exp2(S^T c - lse2) (x dropout mask), dS^T = P^T (dP^T mask - delta), written to shared memory as bf16
//          tiles; the softmax scale is applied once, to dK and dQ, at the end
//   dV  += P^T  . dO_i        [128 keys x HD]             TMEM columns [256, 256 + HD)
//   dK  += dS^T . Q_i         [128 keys x HD]             TMEM columns [384, 384 + HD)
//   dQ   = dS . K             [128 queries x HD]          TMEM columns [128, 128 + HD), once per PAIR of query blocks
// The dS^T tiles of two consecutive query blocks sit side by side in shared memory as the two 64-column chunks of
// one [128 keys][128 queries] tile; read MN-major, that tile is the A operand dS of the dQ product with M = 128, so
// the dQ product runs at the full tile width.  Its result is one key block's share of dQ.  Four drain warps (one per
// TMEM lane quarter) copy it to shared memory and add it to an fp32 accumulator [batch, head, 128-query tile][128][HD]
// in global memory with bulk tensor reductions (cp.reduce.async.bulk.tensor ... add): the additions run in the L2 and
// leave the load/store units of the SM to the math warps.  A small kernel scales the accumulator and writes the bf16
// dQ matrix afterwards.  The order in which the key blocks add their shares is not fixed, so dQ can differ in the
// last bit from run to run; the two-kernel backward stays available for bitwise-reproducible runs.
//
// Order of the tensor-core work (one issuing thread; products retire in issue order).  While the math warps work on
// block i, the issuing thread queues: dV of block i - 1 (frees the single P^T buffer early), then S^T / dP^T of block
// i + 1 (the math warps have copied block i into registers and released the TMEM buffers: sdp_free), then dQ of the
// pair that block i - 1 completed and dK of block i - 1.  So the next block's scores are never queued behind more
// than four small products, and everything the math warps wait for was issued a whole block earlier.
#include "attention_device.cuh"

namespace ssb {

int make_tma_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                     uint32_t box_rows, uint32_t box_cols);
int make_tma_2d_f32(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

namespace {

using namespace attn;

constexpr int kDrainWarps = 4;  // one per TMEM lane quarter
constexpr int kFusedThreads = kAttnThreads + 32 * kDrainWarps;

template <int HD>
struct FusedCfg {
  static constexpr int kCh = HD / 64;
  static constexpr int kKvTile = 128 * HD * 2;   // K_j / V_j, resident
  static constexpr int kQStages = 3;
  static constexpr int kQTile = 64 * HD * 2;     // Q_i / dO_i, kQStages stages each
  static constexpr int kPBytes = 128 * 64 * 2;   // P^T (one buffer), dS^T (two chunks = one pair tile)
  static constexpr int kStageBytes = 32 * 128;   // per drain warp: 32 rows x 32 floats, swizzled like a TMA tile
  static constexpr int kSmem = 2 * kKvTile + 2 * kQStages * kQTile + 3 * kPBytes + kDrainWarps * kStageBytes + 1024 + 256;
  static constexpr int kTmemCols = 512;
  static constexpr int kColS = 0, kColDP = 64, kColDQ = 128, kColDV = 256, kColDK = 384;
};

template <int HD, bool DROPOUT, bool BIAS>
__global__ void __launch_bounds__(kFusedThreads, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_acc, const AttnParams p) {
  using Cfg = FusedCfg<HD>;
  constexpr int CH = Cfg::kCh;
  constexpr int QS = Cfg::kQStages;
  constexpr int OC = HD / 4;  // accumulator columns per math group
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::kKvTile;
  uint8_t* sQ = sV + Cfg::kKvTile;       // QS stages
  uint8_t* sdO = sQ + QS * Cfg::kQTile;  // QS stages
  uint8_t* sPt = sdO + QS * Cfg::kQTile;
  uint8_t* sdSt = sPt + Cfg::kPBytes;    // two chunks: query block parity
  uint8_t* sStage = sdSt + 2 * Cfg::kPBytes;  // kDrainWarps x 4 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStage + kDrainWarps * Cfg::kStageBytes);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // 3
  uint64_t* qdo_empty = bars + 4;    // 3: dK of that stage's block retired (the last reader of Q_i, dO_i)
  uint64_t* s_full = bars + 7;       // 1
  uint64_t* sdp_free = bars + 8;     // 1 (one arrival per math warp): S^T / dP^T copied to registers
  uint64_t* p_full = bars + 9;       // 1 (one arrival per math warp)
  uint64_t* pv_done = bars + 10;     // 1: dV of a block retired (P^T free)
  uint64_t* dk_done = bars + 11;     // 2 (block parity): dK of a block retired (that dS^T chunk free of dK)
  uint64_t* dq_done = bars + 13;     // 1: dQ of a pair retired (both dS^T chunks free of dQ; accumulator ready)
  uint64_t* dq_empty = bars + 14;    // 1 (one arrival per drain warp): dQ accumulator copied out
  uint64_t* acc_full = bars + 15;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.x;  // early key blocks see the most queries under the causal mask
  const int head = blockIdx.y, b = blockIdx.z;
  const int kv0 = jb * 128;
  const int kv_len = p.kv_lens ? min(p.kv_lens[b], p.SK) : p.SK;
  const int nq = (p.SQ + 63) / 64;
  const int i0 = p.causal ? (kv0 / 64) : 0;  // even: kv0 is a multiple of 128
  const int n_it = (kv0 < kv_len && nq > i0) ? nq - i0 : 0;
  const int n_tiles = (p.SQ + 127) / 128;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < QS; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(sdp_free, kMathWarps);
    mbar_init(p_full, kMathWarps);
    mbar_init(pv_done, 1);
    mbar_init(&dk_done[0], 1);
    mbar_init(&dk_done[1], 1);
    mbar_init(dq_done, 1);
    mbar_init(dq_empty, kDrainWarps);
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_acc);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_dq = tmem_base + Cfg::kColDQ, tmem_dv = tmem_base + Cfg::kColDV, tmem_dk = tmem_base + Cfg::kColDK;

  if (warp == 0) {
    // ------------------------------------------ TMA producer ------------------------------------------
    if (elect_one() && n_it > 0) {
      mbar_arrive_expect_tx(kv_full, 2 * Cfg::kKvTile);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        tma_load_2d(sK + c * 16384, &tm_k, kv_full, p.k_col0 + head * HD + c * 64, b * p.SK + kv0);
        tma_load_2d(sV + c * 16384, &tm_v, kv_full, p.v_col0 + head * HD + c * 64, b * p.SK + kv0);
      }
      Pipe pp;
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        if (!mbar_wait(&qdo_empty[pp.stage], pp.phase ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&qdo_full[pp.stage], 2 * Cfg::kQTile);
        const int row = b * p.SQ + (i0 + it) * 64;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          tma_load_2d(sQ + pp.stage * Cfg::kQTile + c * 8192, &tm_q, &qdo_full[pp.stage],
                      p.q_col0 + head * HD + c * 64, row);
          tma_load_2d(sdO + pp.stage * Cfg::kQTile + c * 8192, &tm_do, &qdo_full[pp.stage],
                      p.o_col0 + head * HD + c * 64, row);
        }
        pp.advance(QS);
      }
      if (!ok) {  // let the copies in flight land before the CTA leaves
        for (uint32_t it = 0; it < (1u << 20); ++it)
          if (mbar_try_wait(kv_full, 0)) break;
        for (int s = 0; s < QS; ++s) {
          const uint32_t armed = (s < pp.stage) ? pp.phase : (pp.phase ^ 1);
          for (uint32_t it = 0; it < (1u << 20); ++it)
            if (mbar_try_wait(&qdo_full[s], armed)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------ MMA issuer --------------------------------------------
    if (elect_one() && n_it > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false, false);   // [keys x queries], reduce over HD
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, HD, false, true);  // [keys x HD], reduce over queries
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, HD, true, true);    // [queries x HD], reduce over keys
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      const uint32_t k = smem_u32(sK), v = smem_u32(sV);
      const uint32_t pt = smem_u32(sPt), dst = smem_u32(sdSt);
      auto issue_sdp = [&](int it) {
        const int qs = it % QS;
        const uint32_t qq = smem_u32(sQ + qs * Cfg::kQTile), dd = smem_u32(sdO + qs * Cfg::kQTile);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offa = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t offb = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16_ss(tmem_base + Cfg::kColS, umma_desc_sw128(k + offa, 16, 1024), umma_desc_sw128(qq + offb, 16, 1024),
                      idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offa = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t offb = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16_ss(tmem_base + Cfg::kColDP, umma_desc_sw128(v + offa, 16, 1024),
                      umma_desc_sw128(dd + offb, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(s_full);
      };
      if (ok) ok = mbar_wait(&qdo_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_sdp(0);
      }
      // step `it` queues the work that can run while the math warps are busy with block it
      for (int it = 0; it <= n_it && ok; ++it) {
        const int j = it - 1;  // the block whose P^T / dS^T the math warps have just delivered
        const int jq = j % QS, jc = j & 1, jt = j >> 1;
        if (j >= 0) {
          if (!mbar_wait(p_full, j & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t dd = smem_u32(sdO + jq * Cfg::kQTile);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)  // 64 queries = 4 steps of 16
            umma_f16_ss(tmem_dv, umma_desc_sw128(pt + kk * 32, 16, 1024), umma_desc_sw128(dd + kk * 2048, 8192, 1024),
                        idesc_acc, (j | kk) != 0);
          umma_commit(pv_done);
        }
        if (it + 1 < n_it) {
          if (!mbar_wait(&qdo_full[(it + 1) % QS], ((it + 1) / QS) & 1, abort_flag)) { ok = false; break; }
          if (!mbar_wait(sdp_free, it & 1, abort_flag)) { ok = false; break; }  // block `it` sits in registers
          tc_fence_after_sync();
          issue_sdp(it + 1);
        }
        if (j >= 0) {
          if (jc == 1 || j == n_it - 1) {
            // dQ of the pair: A = dS^T pair tile read MN-major (M = 128 queries in two 64-query chunks), B = K
            if (jt >= 1 && !mbar_wait(dq_empty, (jt - 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)  // 128 keys = 8 steps of 16
              umma_f16_ss(tmem_dq, umma_desc_sw128(dst + kk * 2048, 16384, 1024),
                          umma_desc_sw128(k + kk * 2048, 16384, 1024), idesc_dq, kk != 0);
            umma_commit(dq_done);
          }
          const uint32_t qq = smem_u32(sQ + jq * Cfg::kQTile);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16_ss(tmem_dk, umma_desc_sw128(dst + jc * 16384 + kk * 32, 16, 1024),
                        umma_desc_sw128(qq + kk * 2048, 8192, 1024), idesc_acc, (j | kk) != 0);
          umma_commit(&qdo_empty[jq]);
          umma_commit(&dk_done[jc]);
        }
      }
      if (ok) umma_commit(acc_full);
    }
  } else if (warp >= 2 + kMathWarps) {
    // ------------- drain warps: dQ tile of every finished pair -> fp32 accumulator in global memory -------------
    const int quarter = warp & 3;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint8_t* stage = sStage + (warp - 2 - kMathWarps) * Cfg::kStageBytes;
    const int n_pairs = (n_it + 1) >> 1;
    const int row0 = ((b * p.NH + head) * n_tiles) * 128 + quarter * 32;
    bool ok = true;
    for (int tt = 0; tt < n_pairs && ok; ++tt) {
      if (!mbar_wait_warp(dq_done, tt & 1, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int tile = (i0 >> 1) + tt;
#pragma unroll
      for (int ch = 0; ch < HD / 32; ++ch) {
        uint32_t rq[32];
        tmem_ld_32x32(tmem_dq + lane_addr + ch * 32, rq);
        tmem_ld_wait();
        if (lane == 0) tma_store_wait_read<0>();  // the previous reduction has read this warp's staging tile
        __syncwarp();
        uint8_t* row = stage + lane * 128;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<uint4*>(row + ((i ^ (lane & 7)) << 4)) =
              make_uint4(rq[4 * i], rq[4 * i + 1], rq[4 * i + 2], rq[4 * i + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_2d(&tm_acc, stage, ch * 32, row0 + tile * 128);
          tma_store_commit();
        }
      }
      tc_fence_before_sync();
      warp_arrive(dq_empty, lane);  // the dQ product of the next pair may overwrite the accumulator
    }
    if (lane == 0) tma_store_wait<0>();  // reductions complete before the CTA's shared memory goes away
  } else {
    // ------------------------------------------ math warps --------------------------------------------
    const int quarter = warp & 3;
    const int g = (warp - 2) >> 2;      // column group: 16 of the 64 queries of a block, HD/4 output columns
    const int r = quarter * 32 + lane;  // key row inside the tile
    const int kv = kv0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float c = p.scale * kLog2e;
    const uint32_t keep8 = dropout_keep8(p.dropout_p);
    const float inv_keep = DROPOUT ? 256.0f / static_cast<float>(keep8) : 1.0f;
    const uint32_t bh_seed = static_cast<uint32_t>(hash64(p.dropout_seed, static_cast<uint64_t>(b) * p.NH + head));
    const uint32_t qquads = (p.SQ + 3) >> 2;
    // per (batch, head) statistics prepared by attn_bwd_prep_kernel: lse2 = LSE log2(e), nd = -rowsum(dO O)
    const float* lse_row = p.LSE + (static_cast<size_t>(b) * p.NH + head) * p.SQ;
    const float* nd_row = p.delta + (static_cast<size_t>(b) * p.NH + head) * p.SQ;
    const bool kv_ok = kv < kv_len;
    const bool stats_vec = (p.SQ & 3) == 0;
    // shared-memory offsets of this thread's two 16-byte pieces of a [128][128 B] swizzled tile row: fixed for the
    // whole kernel (row r, pieces 2 g and 2 g + 1)
    // score bias: bias2[q] = bias_table[head][kv - q + SQ - 1] log2(e); its gradient is dS summed along the diagonals
    const int n_dist = p.SQ + p.SK - 1;
    const float* bias_head = BIAS ? p.bias_table + static_cast<size_t>(head) * n_dist : nullptr;
    float* dbias_head = BIAS ? p.dbias_table + static_cast<size_t>(head) * n_dist : nullptr;
    const uint32_t piece_a = static_cast<uint32_t>(r * 128 + (((2 * g) ^ (r & 7)) << 4));
    const uint32_t piece_b = static_cast<uint32_t>(r * 128 + (((2 * g + 1) ^ (r & 7)) << 4));

    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int cpar = it & 1;
      const int qbase = (i0 + it) * 64 + g * 16;
      // statistics of this thread's 16 queries, requested before the accumulators are ready
      float lse2[16], nd[16];
      if (stats_vec && qbase + 16 <= p.SQ) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(lse_row + qbase) + i);
          const float4 d = __ldg(reinterpret_cast<const float4*>(nd_row + qbase) + i);
          lse2[4 * i] = a.x; lse2[4 * i + 1] = a.y; lse2[4 * i + 2] = a.z; lse2[4 * i + 3] = a.w;
          nd[4 * i] = d.x; nd[4 * i + 1] = d.y; nd[4 * i + 2] = d.z; nd[4 * i + 3] = d.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const bool in = qbase + i < p.SQ;
          lse2[i] = in ? __ldg(lse_row + qbase + i) : INFINITY;
          nd[i] = in ? __ldg(nd_row + qbase + i) : 0.f;
        }
      }
      // dropout: this key's hashes of the four query quads of the step (byte e of hash j decides query 4 j + e)
      uint32_t hq[4];
      if constexpr (DROPOUT) {
#pragma unroll
        for (int j = 0; j < 4; ++j) hq[j] = attn_col_hash(bh_seed, kv, qquads, (qbase >> 2) + j);
      }
      const int qblk0 = (i0 + it) * 64;
      const bool need_mask = (p.causal && kv0 + 127 > qblk0) || qblk0 + 64 > p.SQ || kv0 + 128 > kv_len;
      if (!mbar_wait_warp(s_full, it & 1, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t rs[16], rp[16];
      tmem_ld_32x16(tmem_base + lane_addr + Cfg::kColS + g * 16, rs);
      tmem_ld_32x16(tmem_base + lane_addr + Cfg::kColDP + g * 16, rp);
      tmem_ld_wait();
      tc_fence_before_sync();
      warp_arrive(sdp_free, lane);  // the products of the next query block may overwrite S^T / dP^T now
      uint32_t wp[8], wd[8];
      float dsv[BIAS ? 16 : 1];
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        float pv[2], dv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float shift = -lse2[i + e];
          if constexpr (BIAS) {
            const int d = min(max(kv - (qbase + i + e) + p.SQ - 1, 0), n_dist - 1);
            shift = fmaf(__ldg(bias_head + d), kLog2e, shift);
          }
          const float pr = ex2(fmaf(__uint_as_float(rs[i + e]), c, shift));
          const float dp = __uint_as_float(rp[i + e]);
          if constexpr (DROPOUT) {
            const float mk = keep_byte(hq[(i + e) >> 2], (i + e) & 3, keep8) ? inv_keep : 0.f;
            pv[e] = pr * mk;
            dv[e] = pr * fmaf(dp, mk, nd[i + e]);
          } else {
            pv[e] = pr;
            dv[e] = pr * (dp + nd[i + e]);
          }
        }
        if (need_mask) {  // uniform branch: only blocks on the diagonal or at the ragged ends pay for the tests
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int q = qbase + i + e;
            if (!(kv_ok && q < p.SQ && !(p.causal && kv > q))) pv[e] = dv[e] = 0.f;
          }
        }
        wp[i >> 1] = pack_bf16x2(pv[0], pv[1]);
        wd[i >> 1] = pack_bf16x2(dv[0], dv[1]);
        if constexpr (BIAS) {
          dsv[i] = dv[0];
          dsv[i + 1] = dv[1];
        }
      }
      if constexpr (BIAS) {
        // Gradient of the bias table: dS (before the softmax scale) summed along the diagonals key - query.  Lane l
        // holds key kv and queries qbase .. qbase + 15; the diagonal through (l, i) continues at (l + 1, i + 1), so a
        // running sum handed from lane l + 1 to lane l while i walks down collects a warp's share of every diagonal:
        // at the end lane l holds the diagonal through (l, 0), and the diagonals that leave the warp at lane 0 are
        // flushed as they complete.  47 reductions per warp and step instead of 512.
        float run = 0.f;
#pragma unroll
        for (int i = 15; i >= 0; --i) {
          run = dsv[i] + __shfl_down_sync(0xffffffffu, run, 1) * (lane < 31 ? 1.f : 0.f);
          if (i > 0 && lane == 0) {
            const int d = kv - (qbase + i) + p.SQ - 1;
            if (d >= 0 && d < n_dist) atomicAdd(dbias_head + d, run);
          }
        }
        const int d = kv - qbase + p.SQ - 1;
        if (d >= 0 && d < n_dist) atomicAdd(dbias_head + d, run);
      }
      // P^T: read by dV of the previous block (queued at the start of this block).  This parity's dS^T chunk: read by
      // dK of block it - 2 and by dQ of the previous pair, which reads both chunks and was queued during this block
      // when `it` is even, one block earlier when it is odd (then this thread saw it retire at block it - 1).
      if (it >= 1 && !mbar_wait_warp(pv_done, (it - 1) & 1, abort_flag)) { ok = false; break; }
      if (it >= 2) {
        if (!mbar_wait_warp(&dk_done[cpar], ((it >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
        if (cpar == 0 && !mbar_wait_warp(dq_done, ((it >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
      }
      *reinterpret_cast<uint4*>(sPt + piece_a) = make_uint4(wp[0], wp[1], wp[2], wp[3]);
      *reinterpret_cast<uint4*>(sPt + piece_b) = make_uint4(wp[4], wp[5], wp[6], wp[7]);
      uint8_t* ds_chunk = sdSt + cpar * Cfg::kPBytes;
      *reinterpret_cast<uint4*>(ds_chunk + piece_a) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
      *reinterpret_cast<uint4*>(ds_chunk + piece_b) = make_uint4(wd[4], wd[5], wd[6], wd[7]);
      tc_fence_before_sync();
      fence_proxy_async_smem();
      warp_arrive(p_full, lane);
    }
    if (ok && n_it > 0) ok = mbar_wait(acc_full, 0, abort_flag);
    // tcgen05.ld is warp-collective: the whole warp runs the loads, only the stores are predicated
    ok = __all_sync(0xffffffffu, ok);
    const bool store_row = kv < p.SK;
    if (ok) {
      tc_fence_after_sync();
      __nv_bfloat16* dvrow = reinterpret_cast<__nv_bfloat16*>(p.dV) +
                             (static_cast<size_t>(b) * p.SK + kv) * p.lddv + p.dv_col0 + head * HD + g * OC;
      __nv_bfloat16* dkrow = reinterpret_cast<__nv_bfloat16*>(p.dK) +
                             (static_cast<size_t>(b) * p.SK + kv) * p.lddk + p.dk_col0 + head * HD + g * OC;
      uint32_t rv[OC], rk[OC];
      if (n_it > 0) {
        tmem_ld_cols<OC>(tmem_dv + lane_addr + g * OC, rv);
        tmem_ld_cols<OC>(tmem_dk + lane_addr + g * OC, rk);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < OC; ++i) rv[i] = rk[i] = 0u;
      }
      const float sc = p.scale;
#pragma unroll
      for (int i = 0; i < OC / 8; ++i) {
        uint4 wv, wk;
        wv.x = pack_bf16x2(__uint_as_float(rv[8 * i + 0]), __uint_as_float(rv[8 * i + 1]));
        wv.y = pack_bf16x2(__uint_as_float(rv[8 * i + 2]), __uint_as_float(rv[8 * i + 3]));
        wv.z = pack_bf16x2(__uint_as_float(rv[8 * i + 4]), __uint_as_float(rv[8 * i + 5]));
        wv.w = pack_bf16x2(__uint_as_float(rv[8 * i + 6]), __uint_as_float(rv[8 * i + 7]));
        wk.x = pack_bf16x2(__uint_as_float(rk[8 * i + 0]) * sc, __uint_as_float(rk[8 * i + 1]) * sc);
        wk.y = pack_bf16x2(__uint_as_float(rk[8 * i + 2]) * sc, __uint_as_float(rk[8 * i + 3]) * sc);
        wk.z = pack_bf16x2(__uint_as_float(rk[8 * i + 4]) * sc, __uint_as_float(rk[8 * i + 5]) * sc);
        wk.w = pack_bf16x2(__uint_as_float(rk[8 * i + 6]) * sc, __uint_as_float(rk[8 * i + 7]) * sc);
        if (store_row) {
          reinterpret_cast<uint4*>(dvrow)[i] = wv;
          reinterpret_cast<uint4*>(dkrow)[i] = wk;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicMax(p.status, static_cast<int>(kStatusMbarTimeout));
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// dQ[b, q, head, :] (bf16) = scale * the fp32 accumulator [b, head, tile][128][HD]; one thread per 8 columns.
template <int HD>
__global__ void __launch_bounds__(256)
attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int lddq, int dq_col0, int NH,
                       int SQ, int n_tiles, float scale) {
  constexpr int OCT = HD / 8;
  const int head = blockIdx.y, b = blockIdx.z;
  const int idx = blockIdx.x * 256 + threadIdx.x;
  const int q = idx / OCT, j = idx % OCT;
  if (q >= SQ) return;
  const float* src = acc + ((static_cast<size_t>(b) * NH + head) * n_tiles * 128 + q) * HD + j * 8;
  const float4 lo = *reinterpret_cast<const float4*>(src);
  const float4 hi = *reinterpret_cast<const float4*>(src + 4);
  uint4 w;
  w.x = pack_bf16x2(lo.x * scale, lo.y * scale);
  w.y = pack_bf16x2(lo.z * scale, lo.w * scale);
  w.z = pack_bf16x2(hi.x * scale, hi.y * scale);
  w.w = pack_bf16x2(hi.z * scale, hi.w * scale);
  *reinterpret_cast<uint4*>(dq + (static_cast<size_t>(b) * SQ + q) * lddq + dq_col0 + head * HD + j * 8) = w;
}

// Row statistics in the form the fused kernel consumes: nd[b, h, q] = -sum_d dO O and lse2[b, h, q] = LSE log2(e).
// A warp takes one head and 32 consecutive queries of one sequence.  LPR = HD / 8 lanes read one (token, head) row
// with 16-byte loads, so one load instruction of the warp covers 32 / LPR tokens; after the butterfly sum inside the
// lane group every lane of the group holds the row's result, and lane L keeps token (L % LPR) * (32 / LPR) + L / LPR.
template <int HD>
__global__ void __launch_bounds__(128)
attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, int ldo, int o_col0, const __nv_bfloat16* __restrict__ dout,
                     int lddo, const float* __restrict__ lse, float* __restrict__ nd, float* __restrict__ lse2, int B,
                     int NH, int SQ) {
  constexpr int LPR = HD / 8, TPI = 32 / LPR;
  const int lane = threadIdx.x & 31;
  const int qblocks = (SQ + 31) / 32;
  const long long w = blockIdx.x * 4LL + (threadIdx.x >> 5);
  if (w >= static_cast<long long>(B) * NH * qblocks) return;
  const int qb = static_cast<int>(w % qblocks);
  const int head = static_cast<int>((w / qblocks) % NH);
  const int b = static_cast<int>(w / (static_cast<long long>(qblocks) * NH));
  const int sub = lane % LPR, grp = lane / LPR;
  const size_t col = static_cast<size_t>(o_col0) + head * HD + sub * 8;
  float mine = 0.f;
  uint4 qo[LPR], qd[LPR];
#pragma unroll
  for (int i = 0; i < LPR; ++i) {       // all loads first: 2 * LPR independent 16-byte requests per lane
    const int q = qb * 32 + i * TPI + grp;
    const size_t tok = static_cast<size_t>(b) * SQ + min(q, SQ - 1);
    qo[i] = *reinterpret_cast<const uint4*>(o + tok * ldo + col);
    qd[i] = *reinterpret_cast<const uint4*>(dout + tok * lddo + col);
  }
#pragma unroll
  for (int i = 0; i < LPR; ++i) {
    const float2 a0 = unpack_bf16x2(qo[i].x), a1 = unpack_bf16x2(qo[i].y), a2 = unpack_bf16x2(qo[i].z), a3 = unpack_bf16x2(qo[i].w);
    const float2 g0 = unpack_bf16x2(qd[i].x), g1 = unpack_bf16x2(qd[i].y), g2 = unpack_bf16x2(qd[i].z), g3 = unpack_bf16x2(qd[i].w);
    float t = (a0.x * g0.x + a0.y * g0.y) + (a1.x * g1.x + a1.y * g1.y) + (a2.x * g2.x + a2.y * g2.y) +
              (a3.x * g3.x + a3.y * g3.y);
#pragma unroll
    for (int d = LPR / 2; d >= 1; d >>= 1) t += __shfl_xor_sync(0xffffffffu, t, d);
    if (sub == i) mine = t;
  }
  const int q = qb * 32 + sub * TPI + grp;
  if (q < SQ) {
    const size_t idx = (static_cast<size_t>(b) * NH + head) * SQ + q;
    nd[idx] = -mine;
    lse2[idx] = lse[idx] * kLog2e;
  }
}

template <typename K>
int set_smem(K kernel, int bytes) {
  return static_cast<int>(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

template <int HD, bool DROPOUT, bool BIAS>
int launch_fused(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                 const CUtensorMap& tacc, const AttnParams& p, const float* dq_acc, cudaStream_t stream) {
  static bool done = false;
  int rc;
  if (!done) {
    if ((rc = set_smem(attn_bwd_fused_kernel<HD, DROPOUT, BIAS>, FusedCfg<HD>::kSmem))) return rc;
    done = true;
  }
  const int n_tiles = (p.SQ + 127) / 128;
  dim3 grid_kv((p.SK + 127) / 128, p.NH, p.B);
  attn_bwd_fused_kernel<HD, DROPOUT, BIAS><<<grid_kv, kFusedThreads, FusedCfg<HD>::kSmem, stream>>>(tq, tk, tv, tdo, tacc, p);
  dim3 grid_cv((p.SQ * (HD / 8) + 255) / 256, p.NH, p.B);
  attn_dq_convert_kernel<HD><<<grid_cv, 256, 0, stream>>>(dq_acc, reinterpret_cast<__nv_bfloat16*>(p.dQ), p.lddq,
                                                          p.dq_col0, p.NH, p.SQ, n_tiles, p.scale);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// Floats of fp32 scratch the fused backward needs: the dQ accumulator, then the two row-statistic arrays.
long long attn_bwd_fused_scratch_floats(int B, int NH, int SQ, int HD) {
  return static_cast<long long>(B) * NH * ((SQ + 127) / 128) * 128 * HD + 2LL * B * NH * SQ;
}

// dout shares the layout of O (p.ldo / p.o_col0 describe both).  `scratch` holds attn_bwd_fused_scratch_floats()
// floats, 16-byte aligned; the accumulator part is cleared here, on `stream`.
int attn_bwd_fused_launch(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const void* dout,
                          int lddo, const AttnParams& p, float* scratch, cudaStream_t stream) {
  if (p.HD != 64 && p.HD != 128) return -2;
  if (p.causal && p.SQ != p.SK) return -2;
  // 16-byte granularity everywhere: TMA x coordinates (column offsets of Q / K / V / dO), the 16-byte stores of dK /
  // dV and the bulk reductions of dQ; a misaligned offset would fault on the device instead of failing here
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (p.lddq % 8) || (p.lddk % 8) || (p.lddv % 8) ||
      (p.dq_col0 % 8) || (p.dk_col0 % 8) || (p.dv_col0 % 8) || (p.q_col0 % 8) || (p.k_col0 % 8) || (p.v_col0 % 8))
    return -3;
  int rc;
  const int n_tiles = (p.SQ + 127) / 128;
  const long long acc_rows = static_cast<long long>(p.B) * p.NH * n_tiles * 128;
  const long long acc_floats = acc_rows * p.HD;
  const long long stat_floats = static_cast<long long>(p.B) * p.NH * p.SQ;
  float* dq_acc = scratch;
  float* nd = scratch + acc_floats;
  float* lse2 = nd + stat_floats;
  {
    if ((p.ldo % 8) || (p.o_col0 % 8)) return -3;
    const long long warps = static_cast<long long>(p.B) * p.NH * ((p.SQ + 31) / 32);
    const auto* ob = reinterpret_cast<const __nv_bfloat16*>(p.O);
    const auto* db = reinterpret_cast<const __nv_bfloat16*>(dout);
    const unsigned blocks = static_cast<unsigned>((warps + 3) / 4);
    if (p.HD == 128)
      attn_bwd_prep_kernel<128><<<blocks, 128, 0, stream>>>(ob, p.ldo, p.o_col0, db, lddo, p.LSE, nd, lse2, p.B, p.NH, p.SQ);
    else
      attn_bwd_prep_kernel<64><<<blocks, 128, 0, stream>>>(ob, p.ldo, p.o_col0, db, lddo, p.LSE, nd, lse2, p.B, p.NH, p.SQ);
  }
  if ((rc = static_cast<int>(cudaMemsetAsync(dq_acc, 0, sizeof(float) * acc_floats, stream)))) return rc;
  AttnParams pp = p;
  pp.delta = nd;
  pp.LSE = lse2;
  CUtensorMap tq64, tk128, tv128, tdo64, tacc;
  const uint64_t rq = static_cast<uint64_t>(p.B) * p.SQ, rk = static_cast<uint64_t>(p.B) * p.SK;
  if ((rc = make_tma_2d_bf16(&tq64, q, rq, ldq, ldq, 64, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tdo64, dout, rq, lddo, lddo, 64, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tk128, k, rk, ldk, ldk, 128, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tv128, v, rk, ldv, ldv, 128, 64))) return rc;
  if ((rc = make_tma_2d_f32(&tacc, dq_acc, static_cast<uint64_t>(acc_rows), static_cast<uint64_t>(p.HD), 32))) return rc;
  const bool drop = p.dropout_p > 0.f;
  if (p.bias_table != nullptr) {
    if (p.dbias_table == nullptr) return -2;
    if (p.HD == 128)
      return drop ? launch_fused<128, true, true>(tq64, tk128, tv128, tdo64, tacc, pp, dq_acc, stream)
                  : launch_fused<128, false, true>(tq64, tk128, tv128, tdo64, tacc, pp, dq_acc, stream);
    return drop ? launch_fused<64, true, true>(tq64, tk128, tv128, tdo64, tacc, pp, dq_acc, stream)
                : launch_fused<64, false, true>(tq64, tk128, tv128, tdo64, tacc, pp, dq_acc, stream);
  }
  if (p.HD == 128)
    return drop ? launch_fused<128, true, false>(tq64, tk128, tv128, tdo64, tacc, pp, dq_acc, stream)
                : launch_fused<128, false, false>(tq64, tk128, tv128, tdo64, tacc, pp, dq_acc, stream);
  return drop ? launch_fused<64, true, false>(tq64, tk128, tv128, tdo64, tacc, pp, dq_acc, stream)
              : launch_fused<64, false, false>(tq64, tk128, tv128, tdo64, tacc, pp, dq_acc, stream);
}

}  // namespace ssb
