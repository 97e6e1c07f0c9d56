// Flash attention for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
// Replaces four reference ops and three CUDA extensions at once: ParallelAttentionScoreOp (baddbmm),
// ParallelSoftmaxFusionOp (scaled [causal|masked] softmax), ParallelSoftmaxDropoutOp and
// ParallelContextOp (bmm) -- runtime/megatron/model/flex_ops.py:711-1015 -- without ever writing the
// [b, np, sq, sk] score matrix to memory.
//
// Common layout rules (all three kernels):
//   * every operand tile in shared memory is [64-column chunk][row][128 bytes], written by TMA with
//     the 128-byte swizzle (or by the math threads with the same swizzle for P / dS), so the same
//     tile can be consumed K-major (reduction along the columns) or MN-major (reduction along rows);
//   * one math thread owns one accumulator row (tcgen05.ld 32x32b), so row statistics need no shuffles;
//   * warp 0 = TMA producer, warp 1 = TMEM allocator + MMA issuer, warps 2..5 = math / epilogue.
//
//   forward : CTA = 128 queries of one (batch, head); KV blocks of 128; S double-buffered in TMEM so
//             Q.K^T of block j+1 overlaps the softmax of block j; O accumulated in registers.
//   dK/dV   : CTA = 128 keys; query blocks of 64; S^T = K.Q^T and dP^T = V.dO^T double-buffered,
//             dV += P^T.dO and dK += dS^T.Q accumulate in TMEM.
//   dQ      : CTA = 128 queries; key blocks of 64; dQ += dS.K accumulates in TMEM.
#include "attention_device.cuh"

namespace ssb {

int make_tma_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                     uint32_t box_rows, uint32_t box_cols);

namespace {

using namespace attn;

// =============================================================================================
//                                         FORWARD
// =============================================================================================
// Math work is split by COLUMNS over four groups of four warps: the four warps of a group cover the 128
// accumulator rows (a warp may only read the TMEM lanes 32*(warp%4)..+31), and group g owns columns
// [32g, 32g+32) of every S tile and columns [g*HD/4, (g+1)*HD/4) of the output.  One thread therefore
// handles a quarter of a row; the row maximum is exchanged between the four owners of a row through shared
// memory (bounded mbarrier wait), the row sum is kept as per-thread partials and combined once at the end.
// Sixteen math warps give every SM sub-partition four warps to interleave, which hides the latency of
// the dependent ex2 / convert / pack chains that a single warp per sub-partition cannot.
template <int HD>
struct FwdCfg {
  static constexpr int kCh = HD / 64;
  static constexpr int kTile = 128 * HD * 2;  // Q / K / V tile of 128 rows
  static constexpr int kPBytes = 128 * 128 * 2;
  static constexpr int kXBytes = (2 * 4 * 128 + 4 * 128) * 4;  // row-max exchange (2 buffers) + row-sum partials
  static constexpr int kSmem = kTile * 5 + kPBytes + kXBytes + 1024 + 256;
  static constexpr int kTmemCols = 512;  // S0 [0,128) S1 [128,256) O0 [256,256+HD) O1 [384,384+HD)
};

template <int HD, bool BIAS>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using Cfg = FwdCfg<HD>;
  constexpr int CH = Cfg::kCh;
  constexpr int OC = HD / 4;  // output columns per math group
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::kTile;       // 2 stages
  uint8_t* sV = sK + 2 * Cfg::kTile;   // 2 stages
  uint8_t* sP = sV + 2 * Cfg::kTile;
  float* xmax = reinterpret_cast<float*>(sP + Cfg::kPBytes);  // [2][4 groups][128 rows]
  float* xsum = xmax + 2 * 4 * 128;                           // [4 groups][128 rows]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xmax) + Cfg::kXBytes);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* v_full = bars + 3;      // 2
  uint64_t* k_empty = bars + 5;     // 2  (K is free as soon as Q.K^T of its block retired)
  uint64_t* v_empty = bars + 7;     // 2  (V is free after P.V of its block)
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* p_full = bars + 11;     // 1 (kMathThreads arrivals)
  uint64_t* o_full = bars + 12;     // 2
  uint64_t* o_empty = bars + 14;    // 2 (kMathThreads arrivals)
  uint64_t* x_bar = bars + 16;      // [2][4 quarters], 128 arrivals each
  uint64_t* l_bar = bars + 24;      // [4 quarters], 128 arrivals each
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 28);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heavy (late) query blocks first under the causal mask
  const int head = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * 128;
  const int kv_len = p.kv_lens ? min(p.kv_lens[b], p.SK) : p.SK;
  int n_kv = (kv_len + 127) / 128;
  if (p.causal) n_kv = min(n_kv, qb + 1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&o_full[s], 1);
      mbar_init(&o_empty[s], kMathThreads);
    }
    for (int s = 0; s < 8; ++s) mbar_init(&x_bar[s], 128);
    for (int s = 0; s < 4; ++s) mbar_init(&l_bar[s], 128);
    mbar_init(p_full, kMathThreads);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;  // two buffers, 128 columns apart

  if (warp == 0) {
    if (elect_one()) {
      mbar_arrive_expect_tx(q_full, Cfg::kTile);
#pragma unroll
      for (int c = 0; c < CH; ++c)
        tma_load_2d(sQ + c * 16384, &tm_q, q_full, p.q_col0 + head * HD + c * 64, b * p.SQ + q0);
      Pipe pp;
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        if (!mbar_wait(&k_empty[pp.stage], pp.phase ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[pp.stage], Cfg::kTile);
#pragma unroll
        for (int c = 0; c < CH; ++c)
          tma_load_2d(sK + pp.stage * Cfg::kTile + c * 16384, &tm_k, &k_full[pp.stage],
                      p.k_col0 + head * HD + c * 64, b * p.SK + j * 128);
        if (!mbar_wait(&v_empty[pp.stage], pp.phase ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&v_full[pp.stage], Cfg::kTile);
#pragma unroll
        for (int c = 0; c < CH; ++c)
          tma_load_2d(sV + pp.stage * Cfg::kTile + c * 16384, &tm_v, &v_full[pp.stage],
                      p.v_col0 + head * HD + c * 64, b * p.SK + j * 128);
        pp.advance(2);
      }
      if (!ok) {
        for (uint32_t it = 0; it < (1u << 20); ++it)
          if (mbar_try_wait(q_full, 0)) break;
        for (int s = 0; s < 2; ++s) {
          const uint32_t armed = (s < pp.stage) ? pp.phase : (pp.phase ^ 1);
          for (uint32_t it = 0; it < (1u << 20); ++it)
            if (mbar_try_wait(&k_full[s], armed) && mbar_try_wait(&v_full[s], armed)) break;
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one() && n_kv > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, HD, false, true);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_s = [&](int j) {
        const int st = j & 1;
        const uint32_t a = smem_u32(sQ), bb = smem_u32(sK + st * Cfg::kTile);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_f16_ss(tmem_base + st * 128, umma_desc_sw128(a + off, 16, 1024), umma_desc_sw128(bb + off, 16, 1024),
                      idesc_s, k != 0);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[st]);
      };
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < n_kv) {
          if (!mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          issue_s(j + 1);
        }
        // the output buffer of this block was last used by block j-2: wait until the math warps folded it
        if (j >= 2 && !mbar_wait(&o_empty[st], ((j - 2) >> 1) & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(p_full, j & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&v_full[st], ph, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t a = smem_u32(sP), bb = smem_u32(sV + st * Cfg::kTile);
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // 128 keys = 8 steps of 16
          const uint64_t da = umma_desc_sw128(a + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          const uint64_t db = umma_desc_sw128(bb + k * 2048, 16384, 1024);
          umma_f16_ss(tmem_o + st * 128, da, db, idesc_o, k != 0);
        }
        umma_commit(&v_empty[st]);
        umma_commit(&o_full[st]);
      }
    }
  } else {
    const int quarter = warp & 3;        // TMEM lane quarter this warp may read
    const int g = (warp - 2) >> 2;       // column group
    const int r = quarter * 32 + lane;   // row inside the query tile
    const int q = q0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float c = p.scale * kLog2e;
    const uint32_t keep8 = dropout_keep8(p.dropout_p);
    const float inv_keep = p.dropout_p > 0.f ? 256.0f / static_cast<float>(keep8) : 1.0f;  // applied once, to O
    const uint32_t bh_seed = static_cast<uint32_t>(hash64(p.dropout_seed, static_cast<uint64_t>(b) * p.NH + head));
    const uint32_t qquads = (p.SQ + 3) >> 2;
    const int sub = lane & 3;  // position of this query in its quad: lanes 4t .. 4t+3 share the hashes of a key
    // With a bias the logits are brought into the log2 domain first (x c + bias log2 e) and everything below works
    // on them with a factor of one; without it the raw accumulator is used and the factor is c.
    const float cc = BIAS ? 1.0f : c;
    const float* bias_row = BIAS ? p.bias_table + static_cast<size_t>(head) * (p.SQ + p.SK - 1) + (p.SQ - 1) - min(q, p.SQ - 1)
                                 : nullptr;
    float m = -INFINITY, l = 0.f, alpha_pending = 1.f;
    float o[OC];
#pragma unroll
    for (int i = 0; i < OC; ++i) o[i] = 0.f;
    auto fold = [&](int jj) {  // o = o * alpha_pending + P.V of block jj (already complete)
      uint32_t rr[OC];
      tmem_ld_cols<OC>(tmem_o + (jj & 1) * 128 + lane_addr + g * OC, rr);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < OC; ++i) o[i] = o[i] * alpha_pending + __uint_as_float(rr[i]);
    };
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int st = j & 1;
      if (!mbar_wait_warp(&s_full[st], (j >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int kv0 = j * 128 + g * 32;
      const bool need_mask = (p.causal && kv0 + 31 > q0) || (kv0 + 32 > kv_len);
      uint32_t rr[32];
      tmem_ld_32x32(tmem_base + lane_addr + st * 128 + g * 32, rr);
      tmem_ld_wait();
      float mx = -INFINITY;
      if constexpr (BIAS) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float bv = __ldg(bias_row + min(kv0 + i, p.SK - 1));
          rr[i] = __float_as_uint(fmaf(__uint_as_float(rr[i]), c, bv * kLog2e));
        }
      }
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv = kv0 + i;
          if (kv >= kv_len || (p.causal && kv > q)) rr[i] = 0xff800000u;  // -inf
        }
      }
      {  // four independent chains: a single running maximum would serialise 32 dependent instructions
        float m0 = __uint_as_float(rr[0]), m1 = __uint_as_float(rr[1]), m2 = __uint_as_float(rr[2]), m3 = __uint_as_float(rr[3]);
#pragma unroll
        for (int i = 4; i < 32; i += 4) {
          m0 = fmaxf(m0, __uint_as_float(rr[i]));
          m1 = fmaxf(m1, __uint_as_float(rr[i + 1]));
          m2 = fmaxf(m2, __uint_as_float(rr[i + 2]));
          m3 = fmaxf(m3, __uint_as_float(rr[i + 3]));
        }
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      }
      // exchange the partial maxima of the four owners of this row
      float* xm = xmax + st * 512;
      xm[g * 128 + r] = mx;
      mbar_arrive(&x_bar[st * 4 + quarter]);
      if (!mbar_wait_warp(&x_bar[st * 4 + quarter], (j >> 1) & 1, abort_flag)) { ok = false; break; }
      mx = fmaxf(fmaxf(xm[r], xm[128 + r]), fmaxf(xm[256 + r], xm[384 + r]));
      mx = fmaxf(mx, m);
      const float m_use = (mx == -INFINITY) ? 0.f : mx;  // fully masked so far: keep exponents finite
      const float alpha = ex2((m - m_use) * cc);        // m = -inf -> 0
      const float mc = m_use * cc;
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t w[16];
      // each lane of a query quad hashes 8 of the 32 keys of this step (key = kv0 + 4 jj + sub); the quad exchanges them
      uint32_t hq[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
      if (p.dropout_p > 0.f) {
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) hq[jj] = attn_col_hash(bh_seed, kv0 + 4 * jj + sub, qquads, q >> 2);
      }
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float pe[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          pe[e] = ex2(__uint_as_float(rr[i + e]) * cc - mc);  // masked entries: ex2(-inf) = 0
          rs4[e] += pe[e];                                   // four partial sums: no 32-long dependent chain
        }
        if (p.dropout_p > 0.f) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t h = __shfl_sync(0xffffffffu, hq[i >> 2], (lane & ~3) | e);  // hash of key kv0 + i + e
            pe[e] = keep_byte(h, sub, keep8) ? pe[e] : 0.f;
          }
        }
        w[i >> 1] = pack_bf16x2(pe[0], pe[1]);
        w[(i >> 1) + 1] = pack_bf16x2(pe[2], pe[3]);
      }
      // the single P buffer is free once P.V of the previous block retired
      if (j > 0 && !mbar_wait_warp(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
      store_row32_sw128(sP + (g >> 1) * 16384, r, (g & 1) * 4, w);
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(p_full);
      // fold the previous block's P.V (in the frame of the previous maximum) while the tensor core runs this one
      if (j > 0) {
        tc_fence_after_sync();
        fold(j - 1);
        tc_fence_before_sync();
        mbar_arrive(&o_empty[(j - 1) & 1]);
      }
      alpha_pending = alpha;
      l = l * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
      m = mx;
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok && n_kv > 0) {
      if (__all_sync(0xffffffffu, mbar_wait(&o_full[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, abort_flag))) {
        tc_fence_after_sync();
        fold(n_kv - 1);
      } else {
        ok = false;
      }
    }
    // combine the four partial row sums
    xsum[g * 128 + r] = l;
    mbar_arrive(&l_bar[quarter]);
    if (!mbar_wait(&l_bar[quarter], 0, abort_flag)) ok = false;
    l = (xsum[r] + xsum[128 + r]) + (xsum[256 + r] + xsum[384 + r]);
    if (ok && q < p.SQ) {
      const float inv_l = l > 0.f ? inv_keep / l : 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.O) +
                            (static_cast<size_t>(b) * p.SQ + q) * p.ldo + p.o_col0 + head * HD + g * OC;
#pragma unroll
      for (int i = 0; i < OC / 8; ++i) {
        uint4 w;
        w.x = pack_bf16x2(o[8 * i + 0] * inv_l, o[8 * i + 1] * inv_l);
        w.y = pack_bf16x2(o[8 * i + 2] * inv_l, o[8 * i + 3] * inv_l);
        w.z = pack_bf16x2(o[8 * i + 4] * inv_l, o[8 * i + 5] * inv_l);
        w.w = pack_bf16x2(o[8 * i + 6] * inv_l, o[8 * i + 7] * inv_l);
        reinterpret_cast<uint4*>(orow)[i] = w;
      }
      // rows with no visible key get +inf so that the backward probabilities exp(s - lse) vanish
      if (g == 0)
        p.LSE[(static_cast<size_t>(b) * p.NH + head) * p.SQ + q] =
            l > 0.f ? m * (BIAS ? 1.0f / kLog2e : p.scale) + logf(l) : INFINITY;
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

// =============================================================================================
//                                 BACKWARD: dK, dV
// =============================================================================================
template <int HD>
struct DkvCfg {
  static constexpr int kCh = HD / 64;
  static constexpr int kKvTile = 128 * HD * 2;  // K_j / V_j, resident
  static constexpr int kQStages = 3;
  static constexpr int kQTile = 64 * HD * 2;    // Q_i / dO_i, kQStages stages each
  static constexpr int kPBytes = 128 * 64 * 2;  // P^T / dS^T [128 keys][64 queries], one buffer each
  static constexpr int kSmem = 2 * kKvTile + 2 * kQStages * kQTile + 2 * kPBytes + 1024 + 256;
  // TMEM: S^T0 [0,64) S^T1 [64,128) dP^T0 [128,192) dP^T1 [192,256) dV [256,256+HD) dK [384,384+HD)
  static constexpr int kTmemCols = 512;
};

template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                    const AttnParams p) {
  using Cfg = DkvCfg<HD>;
  constexpr int CH = Cfg::kCh;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::kKvTile;
  constexpr int QS = Cfg::kQStages;
  uint8_t* sQ = sV + Cfg::kKvTile;       // QS stages
  uint8_t* sdO = sQ + QS * Cfg::kQTile;  // QS stages
  uint8_t* sPt = sdO + QS * Cfg::kQTile;
  uint8_t* sdSt = sPt + Cfg::kPBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdSt + Cfg::kPBytes);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // 3
  uint64_t* qdo_empty = bars + 4;    // 3
  uint64_t* s_full = bars + 7;       // 2
  uint64_t* p_full = bars + 9;       // 1 (128 arrivals)
  uint64_t* p_empty = bars + 10;     // 1
  uint64_t* acc_full = bars + 11;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.x;  // early key blocks see the most queries under the causal mask
  const int head = blockIdx.y, b = blockIdx.z;
  const int kv0 = jb * 128;
  const int kv_len = p.kv_lens ? min(p.kv_lens[b], p.SK) : p.SK;
  const int nq = (p.SQ + 63) / 64;
  const int i0 = p.causal ? (kv0 / 64) : 0;
  const int n_it = (kv0 < kv_len && nq > i0) ? nq - i0 : 0;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < QS; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) mbar_init(&s_full[s], 1);
    mbar_init(p_full, kMathThreads);
    mbar_init(p_empty, 1);
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_dv = tmem_base + 256, tmem_dk = tmem_base + 384;

  if (warp == 0) {
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
      if (!ok) {
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
    if (elect_one() && n_it > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false, false);   // [keys x queries], reduce over HD
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, HD, false, true);  // [keys x HD], reduce over queries
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      auto issue_sdp = [&](int it) {
        const int st = it & 1;     // TMEM buffer
        const int qs = it % QS;    // Q / dO stage
        const uint32_t k = smem_u32(sK), v = smem_u32(sV);
        const uint32_t qq = smem_u32(sQ + qs * Cfg::kQTile), dd = smem_u32(sdO + qs * Cfg::kQTile);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offa = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t offb = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16_ss(tmem_base + st * 64, umma_desc_sw128(k + offa, 16, 1024), umma_desc_sw128(qq + offb, 16, 1024),
                      idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offa = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t offb = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16_ss(tmem_base + 128 + st * 64, umma_desc_sw128(v + offa, 16, 1024),
                      umma_desc_sw128(dd + offb, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&s_full[st]);
      };
      if (ok) ok = mbar_wait(&qdo_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_sdp(0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int qs = it % QS;
        if (it + 1 < n_it) {
          if (!mbar_wait(&qdo_full[(it + 1) % QS], ((it + 1) / QS) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          issue_sdp(it + 1);
        }
        if (!mbar_wait(p_full, it & 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t pt = smem_u32(sPt), dst = smem_u32(sdSt);
        const uint32_t qq = smem_u32(sQ + qs * Cfg::kQTile), dd = smem_u32(sdO + qs * Cfg::kQTile);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)  // 64 queries = 4 steps of 16
          umma_f16_ss(tmem_dv, umma_desc_sw128(pt + kk * 32, 16, 1024), umma_desc_sw128(dd + kk * 2048, 8192, 1024),
                      idesc_acc, (it | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_f16_ss(tmem_dk, umma_desc_sw128(dst + kk * 32, 16, 1024), umma_desc_sw128(qq + kk * 2048, 8192, 1024),
                      idesc_acc, (it | kk) != 0);
        umma_commit(&qdo_empty[qs]);
        umma_commit(p_empty);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    const int quarter = warp & 3;
    const int g = (warp - 2) >> 2;      // column group: 16 of the 64 queries of a block, HD/4 output columns
    const int r = quarter * 32 + lane;  // key row inside the tile
    const int kv = kv0 + r;
    constexpr int OC = HD / 4;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float c = p.scale * kLog2e;
    const uint32_t keep8 = dropout_keep8(p.dropout_p);
    const float inv_keep = p.dropout_p > 0.f ? 256.0f / static_cast<float>(keep8) : 1.0f;
    const uint32_t bh_seed = static_cast<uint32_t>(hash64(p.dropout_seed, static_cast<uint64_t>(b) * p.NH + head));
    const uint32_t qquads = (p.SQ + 3) >> 2;
    const float* lse_row = p.LSE + (static_cast<size_t>(b) * p.NH + head) * p.SQ;
    const float* delta_row = p.delta + (static_cast<size_t>(b) * p.NH + head) * p.SQ;
    const bool kv_ok = kv < kv_len;
    const bool stats_vec = (p.SQ & 3) == 0;
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int st = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int qbase = (i0 + it) * 64 + g * 16;
      // statistics of this thread's 16 queries, requested before the accumulators are ready
      float lse2[16], dl[16];
      if (stats_vec && qbase + 16 <= p.SQ) {  // 16-byte loads when the rows of LSE / delta are 16-byte aligned
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(lse_row + qbase) + i);
          const float4 d = __ldg(reinterpret_cast<const float4*>(delta_row + qbase) + i);
          lse2[4 * i] = a.x * kLog2e; lse2[4 * i + 1] = a.y * kLog2e; lse2[4 * i + 2] = a.z * kLog2e; lse2[4 * i + 3] = a.w * kLog2e;
          dl[4 * i] = d.x; dl[4 * i + 1] = d.y; dl[4 * i + 2] = d.z; dl[4 * i + 3] = d.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const bool in = qbase + i < p.SQ;
          lse2[i] = in ? __ldg(lse_row + qbase + i) * kLog2e : INFINITY;
          dl[i] = in ? __ldg(delta_row + qbase + i) : 0.f;
        }
      }
      // blocks strictly below the diagonal and inside both sequences need no per-element validity test
      const int qblk0 = (i0 + it) * 64;
      const bool need_mask = (p.causal && kv0 + 127 > qblk0) || qblk0 + 64 > p.SQ || kv0 + 128 > kv_len;
      if (!mbar_wait_warp(&s_full[st], ph, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t rs[16], rp[16];
      tmem_ld_32x16(tmem_base + lane_addr + st * 64 + g * 16, rs);
      tmem_ld_32x16(tmem_base + lane_addr + 128 + st * 64 + g * 16, rp);
      tmem_ld_wait();
      uint32_t wp[8], wd[8];
      // dropout: this key's hashes of the four query quads of the step
      uint32_t hq[4] = {0u, 0u, 0u, 0u};
      if (p.dropout_p > 0.f) {
#pragma unroll
        for (int j = 0; j < 4; ++j) hq[j] = attn_col_hash(bh_seed, kv, qquads, (qbase >> 2) + j);
      }
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        float pv[2], dv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pr = ex2(__uint_as_float(rs[i + e]) * c - lse2[i + e]);
          float dp = __uint_as_float(rp[i + e]);
          float pd = pr;
          if (p.dropout_p > 0.f) {
            const bool keep = keep_byte(hq[(i + e) >> 2], (i + e) & 3, keep8);
            pd = keep ? pr : 0.f;                  // unscaled: dV is multiplied by 256 / keep8 once, at the end
            dp = keep ? dp * inv_keep : 0.f;
          }
          pv[e] = pd;
          dv[e] = pr * (dp - dl[i + e]) * p.scale;
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
      }
      // the single P^T / dS^T buffer is free once the accumulating MMAs of the previous block retired
      if (it > 0 && !mbar_wait_warp(p_empty, (it - 1) & 1, abort_flag)) { ok = false; break; }
      store_row16_sw128(sPt, r, g * 2, wp);
      store_row16_sw128(sdSt, r, g * 2, wd);
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(p_full);
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
#pragma unroll
      for (int i = 0; i < OC / 8; ++i) {
        uint4 wv, wk;
        wv.x = pack_bf16x2(__uint_as_float(rv[8 * i + 0]) * inv_keep, __uint_as_float(rv[8 * i + 1]) * inv_keep);
        wv.y = pack_bf16x2(__uint_as_float(rv[8 * i + 2]) * inv_keep, __uint_as_float(rv[8 * i + 3]) * inv_keep);
        wv.z = pack_bf16x2(__uint_as_float(rv[8 * i + 4]) * inv_keep, __uint_as_float(rv[8 * i + 5]) * inv_keep);
        wv.w = pack_bf16x2(__uint_as_float(rv[8 * i + 6]) * inv_keep, __uint_as_float(rv[8 * i + 7]) * inv_keep);
        wk.x = pack_bf16x2(__uint_as_float(rk[8 * i + 0]), __uint_as_float(rk[8 * i + 1]));
        wk.y = pack_bf16x2(__uint_as_float(rk[8 * i + 2]), __uint_as_float(rk[8 * i + 3]));
        wk.z = pack_bf16x2(__uint_as_float(rk[8 * i + 4]), __uint_as_float(rk[8 * i + 5]));
        wk.w = pack_bf16x2(__uint_as_float(rk[8 * i + 6]), __uint_as_float(rk[8 * i + 7]));
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

// =============================================================================================
//                                   BACKWARD: dQ
// =============================================================================================
template <int HD>
struct DqCfg {
  static constexpr int kCh = HD / 64;
  static constexpr int kQTile = 128 * HD * 2;   // Q_i / dO_i resident
  static constexpr int kKvStages = 3;
  static constexpr int kKvTile = 64 * HD * 2;   // K_j / V_j, kKvStages stages each
  static constexpr int kSBytes = 128 * 64 * 2;  // dS [128 queries][64 keys], 2 buffers
  static constexpr int kSmem = 2 * kQTile + 2 * kKvStages * kKvTile + 2 * kSBytes + 1024 + 256;
  // TMEM: S0 [0,64) S1 [64,128) dP0 [128,192) dP1 [192,256) dQ [256, 256+HD)
  static constexpr int kTmemCols = 512;
};

template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                   const AttnParams p) {
  using Cfg = DqCfg<HD>;
  constexpr int CH = Cfg::kCh;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + Cfg::kQTile;
  constexpr int KS = Cfg::kKvStages;
  uint8_t* sK = sdO + Cfg::kQTile;       // KS stages
  uint8_t* sV = sK + KS * Cfg::kKvTile;  // KS stages
  uint8_t* sdS = sV + KS * Cfg::kKvTile; // 2 buffers
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + 2 * Cfg::kSBytes);
  uint64_t* q_full = bars;          // 1
  uint64_t* kv_full = bars + 1;     // 3
  uint64_t* kv_empty = bars + 4;    // 3
  uint64_t* s_full = bars + 7;      // 2
  uint64_t* ds_full = bars + 9;     // 2 (128 arrivals)
  uint64_t* ds_empty = bars + 11;   // 2
  uint64_t* acc_full = bars + 13;   // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * 128;
  const int kv_len = p.kv_lens ? min(p.kv_lens[b], p.SK) : p.SK;
  int n_it = (kv_len + 63) / 64;
  if (p.causal) n_it = min(n_it, (q0 + 128) / 64);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&ds_full[s], kMathThreads);
      mbar_init(&ds_empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_dq = tmem_base + 256;

  if (warp == 0) {
    if (elect_one() && n_it > 0) {
      mbar_arrive_expect_tx(q_full, 2 * Cfg::kQTile);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        tma_load_2d(sQ + c * 16384, &tm_q, q_full, p.q_col0 + head * HD + c * 64, b * p.SQ + q0);
        tma_load_2d(sdO + c * 16384, &tm_do, q_full, p.o_col0 + head * HD + c * 64, b * p.SQ + q0);
      }
      Pipe pp;
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        if (!mbar_wait(&kv_empty[pp.stage], pp.phase ^ 1, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&kv_full[pp.stage], 2 * Cfg::kKvTile);
        const int row = b * p.SK + it * 64;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          tma_load_2d(sK + pp.stage * Cfg::kKvTile + c * 8192, &tm_k, &kv_full[pp.stage],
                      p.k_col0 + head * HD + c * 64, row);
          tma_load_2d(sV + pp.stage * Cfg::kKvTile + c * 8192, &tm_v, &kv_full[pp.stage],
                      p.v_col0 + head * HD + c * 64, row);
        }
        pp.advance(KS);
      }
      if (!ok) {
        for (uint32_t it = 0; it < (1u << 20); ++it)
          if (mbar_try_wait(q_full, 0)) break;
        for (int s = 0; s < KS; ++s) {
          const uint32_t armed = (s < pp.stage) ? pp.phase : (pp.phase ^ 1);
          for (uint32_t it = 0; it < (1u << 20); ++it)
            if (mbar_try_wait(&kv_full[s], armed)) break;
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one() && n_it > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false, false);   // [queries x keys], reduce over HD
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, HD, false, true);   // [queries x HD], reduce over keys
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_sdp = [&](int it) {
        const int st = it & 1;     // TMEM buffer
        const int ks = it % KS;    // K / V stage
        const uint32_t qq = smem_u32(sQ), dd = smem_u32(sdO);
        const uint32_t k = smem_u32(sK + ks * Cfg::kKvTile), v = smem_u32(sV + ks * Cfg::kKvTile);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offa = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t offb = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16_ss(tmem_base + st * 64, umma_desc_sw128(qq + offa, 16, 1024), umma_desc_sw128(k + offb, 16, 1024),
                      idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offa = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t offb = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16_ss(tmem_base + 128 + st * 64, umma_desc_sw128(dd + offa, 16, 1024),
                      umma_desc_sw128(v + offb, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&s_full[st]);
      };
      if (ok) ok = mbar_wait(&kv_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_sdp(0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (it + 1 < n_it) {
          if (!mbar_wait(&kv_full[(it + 1) % KS], ((it + 1) / KS) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          issue_sdp(it + 1);
        }
        if (!mbar_wait(&ds_full[st], ph, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t ds = smem_u32(sdS + st * Cfg::kSBytes);
        const uint32_t k = smem_u32(sK + (it % KS) * Cfg::kKvTile);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)  // 64 keys = 4 steps of 16
          umma_f16_ss(tmem_dq, umma_desc_sw128(ds + kk * 32, 16, 1024), umma_desc_sw128(k + kk * 2048, 8192, 1024),
                      idesc_dq, (it | kk) != 0);
        umma_commit(&kv_empty[it % KS]);
        umma_commit(&ds_empty[st]);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    const int quarter = warp & 3;
    const int g = (warp - 2) >> 2;  // column group: 16 of the 64 keys of a block, HD/4 output columns
    const int r = quarter * 32 + lane;
    const int q = q0 + r;
    constexpr int OC = HD / 4;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float c = p.scale * kLog2e;
    const uint32_t keep8 = dropout_keep8(p.dropout_p);
    const float inv_keep = p.dropout_p > 0.f ? 256.0f / static_cast<float>(keep8) : 1.0f;
    const uint32_t bh_seed = static_cast<uint32_t>(hash64(p.dropout_seed, static_cast<uint64_t>(b) * p.NH + head));
    const uint32_t qquads = (p.SQ + 3) >> 2;
    const int sub = lane & 3;  // position of this query in its quad
    const bool q_ok = q < p.SQ;
    const size_t stat_idx = (static_cast<size_t>(b) * p.NH + head) * p.SQ + (q_ok ? q : 0);
    const float lse2 = p.LSE[stat_idx] * kLog2e;
    const float delta = p.delta[stat_idx];
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int st = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      if (!mbar_wait_warp(&s_full[st], ph, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int kvb = it * 64 + g * 16;
      const bool need_mask = (p.causal && it * 64 + 63 > q0) || q0 + 128 > p.SQ || it * 64 + 64 > kv_len;
      uint32_t rs[16], rp[16];
      tmem_ld_32x16(tmem_base + lane_addr + st * 64 + g * 16, rs);
      tmem_ld_32x16(tmem_base + lane_addr + 128 + st * 64 + g * 16, rp);
      tmem_ld_wait();
      uint32_t wd[8];
      // each lane of a query quad hashes 4 of the 16 keys of this step (key = kvb + 4 j + sub); the quad exchanges them
      uint32_t hq[4] = {0u, 0u, 0u, 0u};
      if (p.dropout_p > 0.f) {
#pragma unroll
        for (int j = 0; j < 4; ++j) hq[j] = attn_col_hash(bh_seed, kvb + 4 * j + sub, qquads, q >> 2);
      }
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        const int kv = kvb + i;
        float dsv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pr = ex2(__uint_as_float(rs[i + e]) * c - lse2);
          float dp = __uint_as_float(rp[i + e]);
          if (p.dropout_p > 0.f) {
            const uint32_t h = __shfl_sync(0xffffffffu, hq[i >> 2], (lane & ~3) | e);  // hash of key kv + e
            dp = keep_byte(h, sub, keep8) ? dp * inv_keep : 0.f;
          }
          dsv[e] = pr * (dp - delta) * p.scale;
        }
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (!(q_ok && (kv + e) < kv_len && !(p.causal && (kv + e) > q))) dsv[e] = 0.f;
        }
        wd[i >> 1] = pack_bf16x2(dsv[0], dsv[1]);
        wd[(i >> 1) + 1] = pack_bf16x2(dsv[2], dsv[3]);
      }
      if (!mbar_wait_warp(&ds_empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
      store_row16_sw128(sdS + st * Cfg::kSBytes, r, g * 2, wd);
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(&ds_full[st]);
    }
    if (ok && n_it > 0) ok = mbar_wait(acc_full, 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);  // warp-collective loads below; stores are predicated per row
    if (ok) {
      tc_fence_after_sync();
      __nv_bfloat16* dqrow = reinterpret_cast<__nv_bfloat16*>(p.dQ) +
                             (static_cast<size_t>(b) * p.SQ + q) * p.lddq + p.dq_col0 + head * HD + g * OC;
      uint32_t rq[OC];
      if (n_it > 0) {
        tmem_ld_cols<OC>(tmem_dq + lane_addr + g * OC, rq);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < OC; ++i) rq[i] = 0u;
      }
#pragma unroll
      for (int i = 0; i < OC / 8; ++i) {
        uint4 w;
        w.x = pack_bf16x2(__uint_as_float(rq[8 * i + 0]), __uint_as_float(rq[8 * i + 1]));
        w.y = pack_bf16x2(__uint_as_float(rq[8 * i + 2]), __uint_as_float(rq[8 * i + 3]));
        w.z = pack_bf16x2(__uint_as_float(rq[8 * i + 4]), __uint_as_float(rq[8 * i + 5]));
        w.w = pack_bf16x2(__uint_as_float(rq[8 * i + 6]), __uint_as_float(rq[8 * i + 7]));
        if (q_ok) reinterpret_cast<uint4*>(dqrow)[i] = w;
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

// delta[b, h, q] = sum_d dO[b, q, h, d] * O[b, q, h, d]; one warp per (token, head)
__global__ void __launch_bounds__(128)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, int ldo, int o_col0, const __nv_bfloat16* __restrict__ dout,
                  int lddo, int do_col0, float* __restrict__ delta, int B, int NH, int SQ, int HD) {
  const int lane = threadIdx.x & 31;
  const long long w = blockIdx.x * 4LL + (threadIdx.x >> 5);
  const long long total = static_cast<long long>(B) * SQ * NH;
  if (w >= total) return;
  const int head = static_cast<int>(w % NH);
  const long long tok = w / NH;
  const __nv_bfloat16* orow = o + tok * ldo + o_col0 + head * HD;
  const __nv_bfloat16* drow = dout + tok * lddo + do_col0 + head * HD;
  float s = 0.f;
  for (int d = lane * 2; d < HD; d += 64) {
    const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(orow + d));
    const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(drow + d));
    s += a.x * g.x + a.y * g.y;
  }
  s = warp_sum(s);
  if (lane == 0) {
    const long long bb = tok / SQ, q = tok % SQ;
    delta[(bb * NH + head) * SQ + q] = s;
  }
}

template <typename K>
int set_smem(K kernel, int bytes) {
  return static_cast<int>(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

}  // namespace

// delta[b, h, q] = rowsum(dO * O), the first step of both backward paths.
int attn_delta_launch(const AttnParams& p, const void* dout, int lddo, float* delta, cudaStream_t stream) {
  const long long warps = static_cast<long long>(p.B) * p.SQ * p.NH;
  attn_delta_kernel<<<static_cast<unsigned>((warps + 3) / 4), 128, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(p.O), p.ldo, p.o_col0, reinterpret_cast<const __nv_bfloat16*>(dout), lddo,
      p.o_col0, delta, p.B, p.NH, p.SQ, p.HD);
  return static_cast<int>(cudaGetLastError());
}

// q/k/v: base pointers of the 2-D matrices that hold the heads (see AttnParams); ld in elements.
int attn_fwd_launch(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const AttnParams& p,
                    cudaStream_t stream) {
  if (p.HD != 64 && p.HD != 128) return -2;
  if (p.causal && p.SQ != p.SK) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (p.ldo % 8) || (p.q_col0 % 8) || (p.k_col0 % 8) || (p.v_col0 % 8) ||
      (p.o_col0 % 8))
    return -3;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tma_2d_bf16(&tq, q, static_cast<uint64_t>(p.B) * p.SQ, ldq, ldq, 128, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tk, k, static_cast<uint64_t>(p.B) * p.SK, ldk, ldk, 128, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tv, v, static_cast<uint64_t>(p.B) * p.SK, ldv, ldv, 128, 64))) return rc;
  dim3 grid((p.SQ + 127) / 128, p.NH, p.B);
  auto launch = [&](auto kernel, int smem) -> int {
    int r = set_smem(kernel, smem);   // idempotent and cheap; set on every call so each instantiation is covered
    if (r) return r;
    kernel<<<grid, kAttnThreads, smem, stream>>>(tq, tk, tv, p);
    return static_cast<int>(cudaGetLastError());
  };
  const bool bias = p.bias_table != nullptr;
  if (p.HD == 128)
    return bias ? launch(attn_fwd_kernel<128, true>, FwdCfg<128>::kSmem) : launch(attn_fwd_kernel<128, false>, FwdCfg<128>::kSmem);
  return bias ? launch(attn_fwd_kernel<64, true>, FwdCfg<64>::kSmem) : launch(attn_fwd_kernel<64, false>, FwdCfg<64>::kSmem);
}

// dout shares the layout of O (p.ldo / p.o_col0 describe both).
int attn_bwd_launch(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const void* dout,
                    int lddo, const AttnParams& p, float* delta_scratch, cudaStream_t stream) {
  if (p.HD != 64 && p.HD != 128) return -2;
  if (p.causal && p.SQ != p.SK) return -2;
  if (p.bias_table != nullptr) return -2;  // the score bias exists in the forward and the fused backward kernel only
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (p.lddq % 8) || (p.lddk % 8) || (p.lddv % 8) ||
      (p.dq_col0 % 8) || (p.dk_col0 % 8) || (p.dv_col0 % 8) || (p.q_col0 % 8) || (p.k_col0 % 8) || (p.v_col0 % 8) ||
      (p.ldo % 8) || (p.o_col0 % 8))
    return -3;   // TMA x coordinates and 16-byte stores: every column offset and row pitch in units of 8 elements
  int rc;
  if ((rc = attn_delta_launch(p, dout, lddo, delta_scratch, stream))) return rc;
  AttnParams pp = p;
  pp.delta = delta_scratch;
  CUtensorMap tq64, tk128, tv128, tdo64, tq128, tk64, tv64, tdo128;
  const uint64_t rq = static_cast<uint64_t>(p.B) * p.SQ, rk = static_cast<uint64_t>(p.B) * p.SK;
  if ((rc = make_tma_2d_bf16(&tq64, q, rq, ldq, ldq, 64, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tdo64, dout, rq, lddo, lddo, 64, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tk128, k, rk, ldk, ldk, 128, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tv128, v, rk, ldv, ldv, 128, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tq128, q, rq, ldq, ldq, 128, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tdo128, dout, rq, lddo, lddo, 128, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tk64, k, rk, ldk, ldk, 64, 64))) return rc;
  if ((rc = make_tma_2d_bf16(&tv64, v, rk, ldv, ldv, 64, 64))) return rc;
  dim3 grid_kv((p.SK + 127) / 128, p.NH, p.B), grid_q((p.SQ + 127) / 128, p.NH, p.B);
  if (p.HD == 128) {
    static bool done = false;
    if (!done) {
      if ((rc = set_smem(attn_bwd_dkv_kernel<128>, DkvCfg<128>::kSmem))) return rc;
      if ((rc = set_smem(attn_bwd_dq_kernel<128>, DqCfg<128>::kSmem))) return rc;
      done = true;
    }
    attn_bwd_dkv_kernel<128><<<grid_kv, kAttnThreads, DkvCfg<128>::kSmem, stream>>>(tq64, tk128, tv128, tdo64, pp);
    attn_bwd_dq_kernel<128><<<grid_q, kAttnThreads, DqCfg<128>::kSmem, stream>>>(tq128, tk64, tv64, tdo128, pp);
  } else {
    static bool done = false;
    if (!done) {
      if ((rc = set_smem(attn_bwd_dkv_kernel<64>, DkvCfg<64>::kSmem))) return rc;
      if ((rc = set_smem(attn_bwd_dq_kernel<64>, DqCfg<64>::kSmem))) return rc;
      done = true;
    }
    attn_bwd_dkv_kernel<64><<<grid_kv, kAttnThreads, DkvCfg<64>::kSmem, stream>>>(tq64, tk128, tv128, tdo64, pp);
    attn_bwd_dq_kernel<64><<<grid_q, kAttnThreads, DqCfg<64>::kSmem, stream>>>(tq128, tk64, tv64, tdo128, pp);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ssb
