// tcgen05 forward block kernel for sm_100a: one online-softmax update of the carried
// state (o, m, l) with one K/V block, bf16 inputs, head dim 64 or 128.  It computes what
// fwd_block / _fwd_kernel of the reference compute (ring_attention/ring_kernel.py:41-199,
// math of ring.py:58-76).
//
// One CTA owns two 128-row query tiles and walks the K/V tiles of the block:
//   warp 8   : TMA producer   (Q once, then K and V tiles into 2-stage rings)
//   warp 9   : MMA issuer     (S = Q K^T and O += P V as tcgen05.mma, accumulators in TMEM)
//   warps 0-3: softmax of query tile 0 (thread = row: TMEM lane)
//   warps 4-7: softmax of query tile 1
// The two query tiles alternate on the tensor pipe: while the softmax warps of one tile
// turn S into P, the MMAs of the other tile run.  P is written back over S in TMEM as
// packed bf16 and is the A operand of the PV MMA; V is read MN-major straight from the
// K/V layout, so nothing is transposed.  Running max / sum live in registers; O in TMEM
// is rescaled only when the row max grows by more than 2^8, and the carried O of earlier
// ring steps is folded in once, in the epilogue.
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).
#include <cstdio>
#include <cstring>
#include <mutex>

#include "host_util.h"
#include "tc_common.cuh"

namespace ra {

namespace {

using namespace ptx;

constexpr int kFwdThreads = 320;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;  // log2 units: P stays below 2^8
// Of every 16 column pairs of the softmax, how many get their exponentials from the polynomial
// on the FMA pipe (the others use ex2 on the special-function unit).
#ifndef RA_FWD_POLY_PAIRS
#define RA_FWD_POLY_PAIRS 5
#endif
constexpr int kPolyPairs = RA_FWD_POLY_PAIRS;

struct FwdTcParams {
  CUtensorMap map_q, map_k, map_v;
  FwdParams p;
  const TileMeta* meta_q;   // [b][n_q_tiles]  (NULL when there is no mask)
  const TileMeta* meta_kv;  // [b][n_kv_tiles]
  int n_q_tiles, n_kv_tiles;
  unsigned int* status;
};

enum Bar {
  Q_FULL0 = 0, Q_FULL1, K_FULL0, K_FULL1, K_EMPTY0, K_EMPTY1, V_FULL0, V_FULL1, V_EMPTY0, V_EMPTY1,
  S_FULL0, S_FULL1, P_FULL0, P_FULL1, O_FULL, NUM_BARS
};

template <int D>
__global__ void __launch_bounds__(kFwdThreads, 1) tc_fwd_kernel(const __grid_constant__ FwdTcParams P) {
  constexpr int TILE_BYTES = kTileRows * D * 2;
  constexpr int PANELS = D / 64;           // 64-element (128-byte) panels per row
  constexpr int PANEL_BYTES = kTileRows * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + 2 * TILE_BYTES;
  uint8_t* sV = sK + 2 * TILE_BYTES;
  uint16_t* list = reinterpret_cast<uint16_t*>(sV + 2 * TILE_BYTES);
  uint8_t* codes = reinterpret_cast<uint8_t*>(list + kMaxTiles);  // [kMaxTiles] class of each K/V tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(codes + kMaxTiles);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  int* count_slot = reinterpret_cast<int*>(tmem_slot + 2);

  const FwdParams& p = P.p;
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int bh_count = p.b * p.h;
  const int n_pairs = (P.n_q_tiles + 1) / 2;
  const int bh = blockIdx.x % bh_count;
  const int pair = n_pairs - 1 - blockIdx.x / bh_count;  // heaviest causal rows first
  const int hh = bh % p.h, bb = bh / p.h;
  const int qt0 = pair * 2;
  const int ntile = (qt0 + 1 < P.n_q_tiles) ? 2 : 1;
  const uint32_t kinds = p.mod.kinds;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_BARS; ++i) {
      uint32_t cnt = (i == P_FULL0 || i == P_FULL1) ? 128u : 1u;
      mbar_init(&bars[i], cnt);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // List of K/V tiles this CTA visits: index in bits 0-11, "query tile t needs mask arithmetic
  // on it" in bit 12+t, "the tile's positions are contiguous" in bit 14.  Tiles masked for both
  // query tiles are left out.  Every thread classifies its share of the tiles (one round of
  // loads for up to 320 tiles), then warp 0 compacts the classes in order.
  const bool masked = (kinds & kMetaKinds) != 0;
  const bool dense = (kinds & RA_MOD_DENSE) != 0;  // every visited tile takes the in-TMEM pass (it adds the bias tile)
  if (masked) {
    const TileMeta mq0 = P.meta_q[bb * P.n_q_tiles + qt0];
    const TileMeta mq1 = P.meta_q[bb * P.n_q_tiles + qt0 + (ntile - 1)];
    for (int j = threadIdx.x; j < P.n_kv_tiles; j += blockDim.x) {
      const TileMeta mk = P.meta_kv[bb * P.n_kv_tiles + j];
      const int c0 = classify_tiles(kinds, p.mod.window, mq0, mk);
      const int c1 = ntile == 2 ? classify_tiles(kinds, p.mod.window, mq1, mk) : 0;
      const uint32_t code = ((c0 != 1 || dense) ? 1u : 0u) | ((c1 != 1 || dense) ? 2u : 0u) | (mk.pos_contig ? 4u : 0u);
      codes[j] = ((c0 != 0) || (c1 != 0)) ? (uint8_t)(0x80u | code) : (uint8_t)0;  // bit 7: visited
    }
    __syncthreads();
  }
  if (warp == 0) {
    int cnt = 0;
    for (int base = 0; base < P.n_kv_tiles; base += 32) {
      const int j = base + lane;
      bool active = j < P.n_kv_tiles;
      uint32_t code = dense ? 3u : 0u;
      if (active && masked) {
        code = codes[j] & 0x7u;
        active = (codes[j] & 0x80u) != 0;
      }
      const uint32_t vote = __ballot_sync(0xffffffffu, active);
      if (active) list[cnt + __popc(vote & ((1u << lane) - 1))] = (uint16_t)(j | (code << 12));
      cnt += __popc(vote);
    }
    // ALiBi makes the scores grow towards the query's own position: visiting the K/V tiles in
    // ascending order would raise the running max (and rescale O) at nearly every tile for the
    // steeper heads.  Nearest tiles first: the max is found early.  Only the order changes.
    if ((kinds & RA_MOD_ALIBI) && !(kinds & RA_MOD_DENSE)) {
      __syncwarp();
      for (int i = lane; i < cnt / 2; i += 32) {
        const uint16_t a = list[i], z = list[cnt - 1 - i];
        list[i] = z;
        list[cnt - 1 - i] = a;
      }
    }
    if (lane == 0) *count_slot = cnt;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
  const int count = __shfl_sync(0xffffffffu, *count_slot, 0);
  const uint32_t tmem_S[2] = {tmem_base, tmem_base + 128};
  const uint32_t tmem_O[2] = {tmem_base + 256, tmem_base + 256 + D};

  if (warp == 8) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&P.map_q);
      prefetch_tensormap(&P.map_k);
      prefetch_tensormap(&P.map_v);
      for (int t = 0; t < ntile; ++t) {
        mbar_arrive_expect_tx(&bars[Q_FULL0 + t], TILE_BYTES);
        for (int pn = 0; pn < PANELS; ++pn)
          tma_load_4d(sQ + t * TILE_BYTES + pn * PANEL_BYTES, &P.map_q, &bars[Q_FULL0 + t], pn * 64, hh,
                      (qt0 + t) * kTileRows, bb);
      }
      for (int i = 0; i < count; ++i) {
        const int j = list[i] & 0xFFF, s = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&bars[K_EMPTY0 + s], ph ^ 1, abort_flag, P.status, kStFwdProducer)) break;
        mbar_arrive_expect_tx(&bars[K_FULL0 + s], TILE_BYTES);
        for (int pn = 0; pn < PANELS; ++pn)
          tma_load_4d(sK + s * TILE_BYTES + pn * PANEL_BYTES, &P.map_k, &bars[K_FULL0 + s], pn * 64, hh,
                      j * kTileRows, bb);
        if (!mbar_wait(&bars[V_EMPTY0 + s], ph ^ 1, abort_flag, P.status, kStFwdProducer)) break;
        mbar_arrive_expect_tx(&bars[V_FULL0 + s], TILE_BYTES);
        for (int pn = 0; pn < PANELS; ++pn)
          tma_load_4d(sV + s * TILE_BYTES + pn * PANEL_BYTES, &P.map_v, &bars[V_FULL0 + s], pn * 64, hh,
                      j * kTileRows, bb);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------ MMA issuer
    if (count > 0) {  // every lane runs this loop; one elected lane issues each instruction
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      // low descriptor words of the operand tiles; one stage / query tile further is +TILE_BYTES/16
      const uint32_t q_lo = desc_lo(smem_u32(sQ), 16), k_lo = desc_lo(smem_u32(sK), 16);
      const uint32_t v_lo = desc_lo(smem_u32(sV), PANEL_BYTES);  // V is read MN-major: panels 16 KB apart
      bool ok = true;
      auto issue_s = [&](int t, int stage) {
        const uint32_t a0 = q_lo + t * (TILE_BYTES >> 4), b0 = k_lo + stage * (TILE_BYTES >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          constexpr int kPanel16 = PANEL_BYTES >> 4;
          const uint32_t off = (kk >> 2) * kPanel16 + (kk & 3) * 2;
          mma_ss_warp(tmem_S[t], desc_from_lo(a0 + off), desc_from_lo(b0 + off), idesc_qk, kk > 0);
        }
        tc_commit_warp(&bars[S_FULL0 + t]);
      };
      auto issue_pv = [&](int t, int stage, bool first_tile) {
        const uint32_t b0 = v_lo + stage * (TILE_BYTES >> 4);
#pragma unroll
        for (int kk = 0; kk < kTileRows / 16; ++kk)
          mma_ts_warp(tmem_O[t], tmem_S[t] + kk * 8, desc_from_lo(b0 + kk * (2048 >> 4)), idesc_pv,
                 (!first_tile) || kk > 0);
      };
      for (int t = 0; t < ntile && ok; ++t)
        ok = __all_sync(0xffffffffu, mbar_wait(&bars[Q_FULL0 + t], 0, abort_flag, P.status, kStFwdMma));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars[K_FULL0], 0, abort_flag, P.status, kStFwdMma));
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < ntile; ++t) issue_s(t, 0);
        tc_commit_warp(&bars[K_EMPTY0]);
      }
      for (int i = 0; i < count && ok; ++i) {
        const int s = i & 1, sn = (i + 1) & 1;
        const uint32_t ph = (i >> 1) & 1, phn = ((i + 1) >> 1) & 1;
        const bool has_next = i + 1 < count;
        if (has_next && !(ok = __all_sync(0xffffffffu, mbar_wait(&bars[K_FULL0 + sn], phn, abort_flag, P.status, kStFwdMma)))) break;
        if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[V_FULL0 + s], ph, abort_flag, P.status, kStFwdMma)))) break;
        for (int t = 0; t < ntile; ++t) {
          if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[P_FULL0 + t], i & 1, abort_flag, P.status, kStFwdMma)))) break;
          tc_fence_after();
          issue_pv(t, s, i == 0);
          if (t == ntile - 1) tc_commit_warp(&bars[V_EMPTY0 + s]);
          if (has_next) {
            issue_s(t, sn);
            if (t == ntile - 1) tc_commit_warp(&bars[K_EMPTY0 + sn]);
          }
        }
      }
      if (ok) tc_commit_warp(&bars[O_FULL]);
    }
  } else if (warp < 4 * ntile) {
    // ------------------------------------------------------------ softmax + epilogue
    const int t = warp >> 2;
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const int q_row = (qt0 + t) * kTileRows + row_in_tile;
    const int64_t state_row = ((int64_t)bb * p.h + hh) * p.lq + q_row;
    const float scale2 = p.scale * kLog2e;

    float m_ref = -INFINITY, l_run = 0.f, alpha_total = 1.f;
    if (!p.first) {
      m_ref = p.m[state_row] * kLog2e;
      l_run = p.l[state_row];
    }
    float m_true = m_ref;
    int32_t qpos = 0, qseg = 0;
    bool qpre = false;
    if (p.mod.q_pos) qpos = p.mod.q_pos[(int64_t)bb * p.lq + q_row];
    if (p.mod.q_seg) qseg = p.mod.q_seg[(int64_t)bb * p.lq + q_row];
    if (p.mod.q_pre) qpre = p.mod.q_pre[(int64_t)bb * p.lq + q_row] != 0;
    const bool alibi = (kinds & RA_MOD_ALIBI) != 0;
    bool ok = true;

    const float alibi_over_scale = alibi ? p.mod.slopes[hh] / p.scale : 0.f;
    const float slope2 = alibi ? p.mod.slopes[hh] * kLog2e : 0.f;
    // first position of the K/V tile the loop is about to visit, read one tile ahead
    const bool has_pos = p.mod.kv_pos != nullptr;
    int32_t k0_next = (has_pos && count > 0) ? p.mod.kv_pos[(int64_t)bb * p.lk + (int64_t)(list[0] & 0xFFF) * kTileRows] : 0;
    for (int i = 0; i < count; ++i) {
      const int j = list[i] & 0xFFF;
      const bool need_mask = ((list[i] >> (12 + t)) & 1) != 0;
      // ALiBi over a tile of contiguous key positions with nothing masked is two FMAs per score
      // in registers; every other ALiBi tile takes the in-TMEM pass below
      const bool kv_contig = ((list[i] >> 14) & 1) != 0;
      const bool alibi_inline = alibi && !need_mask && kv_contig;
      const int32_t k0 = k0_next;
      if (has_pos && i + 1 < count) k0_next = p.mod.kv_pos[(int64_t)bb * p.lk + (int64_t)(list[i + 1] & 0xFFF) * kTileRows];
      if (!(ok = mbar_wait(&bars[S_FULL0 + t], i & 1, abort_flag, P.status, kStFwdSoftmax))) break;
      tc_fence_after();
      if (need_mask || (alibi && !alibi_inline)) {  // tiles that mix visible and masked pairs, ALiBi over scattered positions
        const int64_t kv0 = (int64_t)bb * p.lk + (int64_t)j * kTileRows;
        fixup_scores_tmem<true>(tmem_S[t] + lane_off, kTileRows, need_mask ? kinds : (kinds & RA_MOD_ALIBI),
                                p.mod.window, alibi_over_scale, qpos, qseg, qpre,
                                p.mod.kv_pos ? p.mod.kv_pos + kv0 : nullptr, p.mod.kv_seg ? p.mod.kv_seg + kv0 : nullptr,
                                p.mod.kv_pre ? p.mod.kv_pre + kv0 : nullptr, k0, kv_contig,
                                dense ? p.mod.bias + (int64_t)bb * p.mod.bsb + (int64_t)hh * p.mod.bsh +
                                            (int64_t)q_row * p.mod.bsq + (int64_t)j * kTileRows
                                      : nullptr,
                                1, 1.f / p.scale);
      }
      uint32_t r[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tmem_S[t] + lane_off + c * 32, r[c]);
      tc_wait_ld();
      // sc: what is left to multiply the register values by (the ALiBi form has the scale in already)
      float sc = scale2;
      if (alibi_inline) {
        // scale * s - slope * (q_pos - kv_pos), times log2(e): the bias of ring_test.py-style ALiBi
        // callables, with kv_pos = k0 + column; the differences are exact in fp32
        const float r_i = slope2 * (float)(k0 - qpos);
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e)
            r[c][e] = __float_as_uint(fmaf(slope2, (float)(c * 32 + e), fmaf(__uint_as_float(r[c][e]), scale2, r_i)));
        sc = 1.f;
      }
      // raw scores; the scale is positive, so it commutes with max.  Four independent chains of
      // three-input maxima instead of one chain of 128 dependent operations.
      float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int e = 0; e < 32; e += 2) mxa[c] = max3(mxa[c], __uint_as_float(r[c][e]), __uint_as_float(r[c][e + 1]));
      const float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));
      const float m_new = fmaxf(m_true, mx * sc);
      m_true = m_new;
      const bool need = (m_new > m_ref + kRescaleThreshold) || (m_ref == -INFINITY && m_new != -INFINITY);
      if (__any_sync(0xffffffffu, need)) {
        const float alpha = (m_ref == -INFINITY) ? 0.f : ex2(m_ref - m_new);
        m_ref = m_new;
        l_run *= alpha;
        alpha_total *= alpha;
        if (i > 0) {  // O of this tile holds the sum over the tiles before this one
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {
            uint32_t o[16];
            tmem_ld16(tmem_O[t] + lane_off + c * 16, o);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st16(tmem_O[t] + lane_off + c * 16, o);
          }
        }
      }
      const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
      // p = 2^(s * sc - m) on pairs of columns: the first kPolyPairs of every 16 pairs take the
      // polynomial on the FMA pipe, the rest the special-function unit, so that the two pipes
      // finish together; one packed sum per 32-column chunk
      const uint64_t sc2 = pack2(sc, sc), nm2 = pack2(neg_m, neg_m);
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const uint64_t x2 = fma2(pack2(__uint_as_float(r[c][2 * e]), __uint_as_float(r[c][2 * e + 1])), sc2, nm2);
          float p0, p1;
          if (e < kPolyPairs) {
            exp2_poly2(x2, p0, p1);
          } else {
            float x0, x1;
            unpack2(x2, x0, x1);
            p0 = ex2(x0);
            p1 = ex2(x1);
          }
          sum2[c] = add2(sum2[c], pack2(p0, p1));
          pk[e] = pack_bf16(p0, p1);
        }
        tmem_st16(tmem_S[t] + lane_off + c * 16, pk);
      }
      {
        float s0, s1;
        unpack2(add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3])), s0, s1);
        l_run += s0 + s1;
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&bars[P_FULL0 + t]);
    }

    // Epilogue: fold in the carried state of earlier ring steps, bring (o, m, l) to the
    // exact running max, store.
    if (ok && count > 0) ok = mbar_wait(&bars[O_FULL], 0, abort_flag, P.status, kStFwdSoftmax);
    if (ok) {
      tc_fence_after();
      const float beta = (m_ref == -INFINITY) ? 1.f : ex2(m_ref - m_true);
      const float in_scale = p.first ? 0.f : alpha_total * beta;
      float* o_row = p.o + state_row * D;
      const bool finalize = p.final_out.ptr != nullptr;
      const float l_tot = l_run * beta;
      const float inv_l = 1.f / l_tot;  // l = 0 (a row that saw no key) gives 0 * inf = NaN, as o / l does
      __nv_bfloat16* out_row = finalize ? (__nv_bfloat16*)p.final_out.ptr + (int64_t)bb * p.final_out.sb +
                                              (int64_t)q_row * p.final_out.sl + (int64_t)hh * p.final_out.sh
                                        : nullptr;
#pragma unroll 1
      for (int c = 0; c < D / 8; ++c) {
        uint32_t o[8];
        if (count > 0) {
          tmem_ld8(tmem_O[t] + lane_off + c * 8, o);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = 0u;
        }
        float val[8];
#pragma unroll
        for (int e = 0; e < 8; e += 4) {
          float4 prev = make_float4(0.f, 0.f, 0.f, 0.f);
          if (!p.first) prev = *reinterpret_cast<const float4*>(o_row + c * 8 + e);
          val[e] = __uint_as_float(o[e]) * beta + prev.x * in_scale;
          val[e + 1] = __uint_as_float(o[e + 1]) * beta + prev.y * in_scale;
          val[e + 2] = __uint_as_float(o[e + 2]) * beta + prev.z * in_scale;
          val[e + 3] = __uint_as_float(o[e + 3]) * beta + prev.w * in_scale;
        }
        if (finalize) {
          uint4 w;
          w.x = pack_bf16(val[0] * inv_l, val[1] * inv_l);
          w.y = pack_bf16(val[2] * inv_l, val[3] * inv_l);
          w.z = pack_bf16(val[4] * inv_l, val[5] * inv_l);
          w.w = pack_bf16(val[6] * inv_l, val[7] * inv_l);
          *reinterpret_cast<uint4*>(out_row + c * 8) = w;
        } else {
          *reinterpret_cast<float4*>(o_row + c * 8) = make_float4(val[0], val[1], val[2], val[3]);
          *reinterpret_cast<float4*>(o_row + c * 8 + 4) = make_float4(val[4], val[5], val[6], val[7]);
        }
      }
      if (finalize) {
        if (p.final_lse) p.final_lse[state_row] = m_true * (1.f / kLog2e) + logf(l_tot);
      } else {
        p.m[state_row] = m_true * (1.f / kLog2e);
        p.l[state_row] = l_tot;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// -----------------------------------------------------------------------------------------
__global__ void tile_meta_kernel(TileMeta* __restrict__ out, const int32_t* __restrict__ pos,
                                 const int32_t* __restrict__ seg, const uint8_t* __restrict__ pre, int len) {
  // one warp per tile: 4 tokens per lane
  const int n_tiles = len / kTileRows;
  const int tile = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31, bb = blockIdx.y;
  if (tile >= n_tiles) return;
  const int64_t base = (int64_t)bb * len + (int64_t)tile * kTileRows;
  int pmin = INT32_MAX, pmax = INT32_MIN, smin = INT32_MAX, smax = INT32_MIN, any = 0, all = 1, contig = 1;
  const int p0 = pos ? pos[base] : 0;
  for (int e = lane; e < kTileRows; e += 32) {
    if (pos) {
      int v = pos[base + e];
      pmin = min(pmin, v);
      pmax = max(pmax, v);
      contig &= (v == p0 + e) ? 1 : 0;
    }
    if (seg) {
      int v = seg[base + e];
      smin = min(smin, v);
      smax = max(smax, v);
    }
    if (pre) {
      int v = pre[base + e] != 0;
      any |= v;
      all &= v;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    pmin = min(pmin, __shfl_xor_sync(0xffffffffu, pmin, o));
    pmax = max(pmax, __shfl_xor_sync(0xffffffffu, pmax, o));
    smin = min(smin, __shfl_xor_sync(0xffffffffu, smin, o));
    smax = max(smax, __shfl_xor_sync(0xffffffffu, smax, o));
    any |= __shfl_xor_sync(0xffffffffu, any, o);
    all &= __shfl_xor_sync(0xffffffffu, all, o);
    contig &= __shfl_xor_sync(0xffffffffu, contig, o);
  }
  if (lane == 0) {
    TileMeta m;
    m.pos_min = pos ? pmin : 0;
    m.pos_max = pos ? pmax : 0;
    m.seg_min = seg ? smin : 0;
    m.seg_max = seg ? smax : 0;
    m.pre_any = pre ? any : 0;
    m.pre_all = pre ? all : 0;
    m.pos_contig = pos ? contig : 0;
    m.pad1 = 0;
    out[(int64_t)bb * n_tiles + tile] = m;
  }
}

__device__ unsigned int g_status_word = 0;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

template <int D>
cudaError_t launch_fwd(const FwdTcParams& P, cudaStream_t s) {
  constexpr size_t kSmem = 6 * kTileRows * D * 2 + kMaxTiles * 3 + NUM_BARS * 8 + 64 + 1024;
  constexpr size_t kRequest = kSmem < 120 * 1024 ? 120 * 1024 : kSmem;  // one CTA per SM: it owns all of TMEM
  auto kern = tc_fwd_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRequest);
  if (e != cudaSuccess) return e;
  const int n_pairs = (P.n_q_tiles + 1) / 2;
  kern<<<n_pairs * P.p.b * P.p.h, kFwdThreads, kRequest, s>>>(P);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

cudaError_t scratch_alloc(void** ptr, size_t bytes, cudaStream_t s) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static cudaMemPool_t pools[kMaxDevices] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  cudaMemPool_t pool;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!pools[dev]) {
      cudaMemPoolProps props;
      memset(&props, 0, sizeof(props));
      props.allocType = cudaMemAllocationTypePinned;
      props.handleTypes = cudaMemHandleTypeNone;
      props.location.type = cudaMemLocationTypeDevice;
      props.location.id = dev;
      if ((e = cudaMemPoolCreate(&pools[dev], &props)) != cudaSuccess) {
        pools[dev] = nullptr;
        return e;
      }
      uint64_t keep = UINT64_MAX;
      if ((e = cudaMemPoolSetAttribute(pools[dev], cudaMemPoolAttrReleaseThreshold, &keep)) != cudaSuccess) return e;
    }
    pool = pools[dev];
  }
  return cudaMallocFromPoolAsync(ptr, bytes, pool, s);
}

unsigned int* device_status_word() {
  // looked up once per device, with that device current (the symbol's name is a host-side
  // handle, not an address a kernel can use)
  constexpr int kMaxDevices = 64;
  static unsigned int* cache[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  unsigned int* ptr = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
  if (!ptr) {
    if (cudaGetSymbolAddress((void**)&ptr, g_status_word) != cudaSuccess || !ptr) return nullptr;
    __atomic_store_n(&cache[dev], ptr, __ATOMIC_RELEASE);
  }
  return ptr;
}

bool make_tile_map(CUtensorMap* map, const TensorView& t, int b, int len, int h, int d, int box_rows,
                   const char** why) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    *why = "cuTensorMapEncodeTiled is not available from this driver";
    return false;
  }
  const cuuint64_t row_bytes = (cuuint64_t)d * 2;
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)h, (cuuint64_t)len, (cuuint64_t)b};
  cuuint64_t strides[3] = {h > 1 ? (cuuint64_t)t.sh * 2 : row_bytes, len > 1 ? (cuuint64_t)t.sl * 2 : row_bytes,
                           b > 1 ? (cuuint64_t)t.sb * 2 : row_bytes};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(t.ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    *why = "the driver refused the tensor map for these strides";
    return false;
  }
  return true;
}

cudaError_t launch_tile_meta(TileMeta* out, const int32_t* pos, const int32_t* seg, const uint8_t* pre, int b,
                             int len, cudaStream_t s) {
  const int n_tiles = len / kTileRows;
  dim3 grid((n_tiles + 7) / 8, b);
  tile_meta_kernel<<<grid, 256, 0, s>>>(out, pos, seg, pre, len);
  count_launch();
  return cudaGetLastError();
}

static bool aligned16(const TensorView& t) {
  return (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 && (t.sb % 8) == 0 && (t.sl % 8) == 0 && (t.sh % 8) == 0;
}

const char* tc_fwd_unsupported_reason(const FwdParams& p, int dtype) {
  if (dtype != RA_DTYPE_BF16) return "inputs are not bf16";
  if (p.dk != p.dv || (p.dk != 64 && p.dk != 128)) return "head dims must be equal and 64 or 128";
  if (p.lq % kTileRows || p.lk % kTileRows) return "lq and lk must be multiples of 128";
  if (p.lq / kTileRows > kMaxTiles || p.lk / kTileRows > kMaxTiles) return "more than 4096 tiles along one axis";
  if ((p.mod.kinds & RA_MOD_DENSE) &&
      ((reinterpret_cast<uintptr_t>(p.mod.bias) & 15) || (p.mod.bsb % 4) || (p.mod.bsh % 4) || (p.mod.bsq % 4)))
    return "the dense bias needs a 16-byte aligned base and strides that are multiples of 4 floats";
  if (!aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v)) return "q/k/v need 16-byte aligned base and strides";
  if (!(p.scale > 0.f)) return "sm_scale must be positive";
  if (p.final_out.ptr && !aligned16(p.final_out)) return "out needs a 16-byte aligned base and strides";
  return nullptr;
}

cudaError_t tc_fwd_block(const FwdParams& p, cudaStream_t s) {
  FwdTcParams P;
  memset(&P, 0, sizeof(P));
  P.p = p;
  P.n_q_tiles = p.lq / kTileRows;
  P.n_kv_tiles = p.lk / kTileRows;
  const char* why = nullptr;
  if (!make_tile_map(&P.map_q, p.q, p.b, p.lq, p.h, p.dk, kTileRows, &why) ||
      !make_tile_map(&P.map_k, p.k, p.b, p.lk, p.h, p.dk, kTileRows, &why) ||
      !make_tile_map(&P.map_v, p.v, p.b, p.lk, p.h, p.dv, kTileRows, &why))
    return cudaErrorNotSupported;
  P.status = device_status_word();
  if (!P.status) return cudaErrorInvalidSymbol;
  TileMeta* meta = nullptr;
  cudaError_t e = cudaSuccess;
  if (p.mod.kinds & kMetaKinds) {
    const size_t n = (size_t)p.b * (P.n_q_tiles + P.n_kv_tiles);
    if ((e = scratch_alloc((void**)&meta, n * sizeof(TileMeta), s)) != cudaSuccess) return e;
    TileMeta* mq = meta;
    TileMeta* mk = meta + (size_t)p.b * P.n_q_tiles;
    if ((e = launch_tile_meta(mq, p.mod.q_pos, p.mod.q_seg, p.mod.q_pre, p.b, p.lq, s)) == cudaSuccess)
      e = launch_tile_meta(mk, p.mod.kv_pos, p.mod.kv_seg, p.mod.kv_pre, p.b, p.lk, s);
    P.meta_q = mq;
    P.meta_kv = mk;
  }
  if (e == cudaSuccess) e = p.dk == 128 ? launch_fwd<128>(P, s) : launch_fwd<64>(P, s);
  if (meta) cudaFreeAsync(meta, s);  // stream-ordered: after the kernels above, also when one failed to launch
  return e;
}

}  // namespace ra

// -----------------------------------------------------------------------------------------
// Forward block for callers that must not allocate.
//
// tc_fwd_block above takes a few kilobytes of scratch from the stream-ordered allocator for
// the per-tile mask summaries.  Some hosts cannot afford that: the handler of an XLA / JAX
// FFI custom call runs while XLA's own allocator holds nearly all of the GPU's memory, so a
// driver allocation made from inside the handler can fail or stall the device; a serving
// process that has handed all free memory to its own arena is in the same position.  For
// them the same kernel is offered with its scratch in a fixed array that is part of the
// library image: every GPU that loads the library holds these 512 KiB until the process
// exits, and nothing is allocated or freed by a call.
//
// All calls share the one array and it keeps whatever the last call wrote.  The summaries
// a call needs are completely rewritten by that call's own first two launches, so nothing
// has to be cleared; but two calls that overlap on the GPU (different streams, or two host
// threads) overwrite each other's summaries.  Callers must serialise them.
// -----------------------------------------------------------------------------------------
namespace ra {

namespace {

constexpr int kStaticMaxTiles = RA_STATIC_MAX_TILES;
static __device__ __align__(256) TileMeta g_static_tile_meta[kStaticMaxTiles];

constexpr int kMaxDevices = 64;

// Device address of the array on the current device.  The array's name is only a host-side
// handle for the symbol; the address a kernel can use has to be asked for, once per device,
// with that device current.
cudaError_t static_tile_meta(TileMeta** out) {
  static TileMeta* cache[kMaxDevices] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  TileMeta* ptr = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
  if (!ptr) {
    void* sym = nullptr;
    e = cudaGetSymbolAddress(&sym, g_static_tile_meta);
    if (e != cudaSuccess) return e;
    if (!sym) return cudaErrorInvalidSymbol;
    ptr = static_cast<TileMeta*>(sym);
    __atomic_store_n(&cache[dev], ptr, __ATOMIC_RELEASE);
  }
  *out = ptr;
  return cudaSuccess;
}

}  // namespace

}  // namespace ra

extern "C" int ra_fwd_block_static(const ra_shape_t* shape, const ra_tensor_t* q, const ra_tensor_t* k,
                                   const ra_tensor_t* v, const ra_score_mod_t* mod, float* o, float* m,
                                   float* l, int first, void* stream) {
  using namespace ra;
  int rc;
  if ((rc = check_shape(shape))) return rc;
  if ((rc = check_tensor(q, "q")) || (rc = check_tensor(k, "k")) || (rc = check_tensor(v, "v"))) return rc;
  if (!o || !m || !l) return fail(-6, "carried state (o, m, l) is NULL");
  FwdTcParams P;
  memset(&P, 0, sizeof(P));
  FwdParams& p = P.p;
  if ((rc = check_mod(mod, &p.mod))) return rc;
  p.q = TensorView{q->ptr, q->stride_b, q->stride_l, q->stride_h};
  p.k = TensorView{k->ptr, k->stride_b, k->stride_l, k->stride_h};
  p.v = TensorView{v->ptr, v->stride_b, v->stride_l, v->stride_h};
  p.o = o;
  p.m = m;
  p.l = l;
  p.b = shape->b;
  p.h = shape->h;
  p.lq = shape->lq;
  p.lk = shape->lk;
  p.dk = shape->dk;
  p.dv = shape->dv;
  p.scale = shape->sm_scale;
  p.first = first ? 1 : 0;
  if (const char* why = tc_fwd_unsupported_reason(p, shape->dtype))
    return fail(-40, "ra_fwd_block_static serves only what the tcgen05 forward takes: %s", why);
  P.n_q_tiles = p.lq / kTileRows;
  P.n_kv_tiles = p.lk / kTileRows;
  // the fixed array holds the tile summaries, which only calls with a mask or ALiBi read
  const bool uses_scratch = (p.mod.kinds & kMetaKinds) != 0;
  const long long tiles = (long long)p.b * (P.n_q_tiles + P.n_kv_tiles);
  if (uses_scratch && tiles > kStaticMaxTiles)
    return fail(-41, "ra_fwd_block_static: b * (lq/128 + lk/128) = %lld tiles exceeds the fixed scratch of %d tiles",
                tiles, kStaticMaxTiles);
  const char* why = nullptr;
  if (!make_tile_map(&P.map_q, p.q, p.b, p.lq, p.h, p.dk, kTileRows, &why) ||
      !make_tile_map(&P.map_k, p.k, p.b, p.lk, p.h, p.dk, kTileRows, &why) ||
      !make_tile_map(&P.map_v, p.v, p.b, p.lk, p.h, p.dv, kTileRows, &why))
    return fail(-42, "ra_fwd_block_static: %s", why);
  P.status = device_status_word();
  if (!P.status) return fail(RA_ERR_CUDA, "status word symbol not found");
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e;
  if (uses_scratch) {
    TileMeta* meta = nullptr;
    if ((e = static_tile_meta(&meta)) != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(static scratch)");
    TileMeta* mq = meta;
    TileMeta* mk = meta + (size_t)p.b * P.n_q_tiles;
    if ((e = launch_tile_meta(mq, p.mod.q_pos, p.mod.q_seg, p.mod.q_pre, p.b, p.lq, s)) != cudaSuccess ||
        (e = launch_tile_meta(mk, p.mod.kv_pos, p.mod.kv_seg, p.mod.kv_pre, p.b, p.lk, s)) != cudaSuccess)
      return fail_cuda(e, "tile summaries");
    P.meta_q = mq;
    P.meta_kv = mk;
  }
  e = p.dk == 128 ? launch_fwd<128>(P, s) : launch_fwd<64>(P, s);
  if (e != cudaSuccess) return fail_cuda(e, "tcgen05 forward block (static scratch)");
  set_last_impl(RA_IMPL_TCGEN05);
  return 0;
}
