// tcgen05 backward block kernel for sm_100a: adds one (Q block, K/V block) pair's
// contribution to dQ, dK, dV; bf16 inputs, head dim 64 or 128.  It computes what
// bwd_block / _bwd_kernel of the reference compute (ring_attention/ring_kernel.py:202-384,
// math of ring.py:140-157), with delta = rowsum(dO * O) precomputed once per backward
// instead of once per ring step (ring_kernel.py:227).
//
// One CTA owns a 128-row K/V tile (dK, dV accumulate in TMEM for the whole kernel) and
// walks the 128-row query tiles.  Everything is computed transposed, so that the thread
// that owns TMEM lane r owns key row r:
//   S^T  = K Q^T          (SS MMA, both operands K-major)            -> TMEM [0,128)
//   dP^T = V dO^T         (SS MMA)                                   -> TMEM [128,256)
//   P^T  = exp2(S^T * c - L * log2 e)            written back over S^T as packed bf16 (TMEM)
//   dS^T = P^T * (dP^T - delta) * scale          written to shared memory as bf16 (128B swizzle)
//          (the per-row terms -L * log2 e and -delta * scale are computed once per backward, and
//           the softmax scale rides on dS^T, so dQ and dK need no further scaling)
//   dV  += P^T dO         (TS MMA: A from TMEM, B = dO read MN-major) -> TMEM [256,256+D)
//   dK  += dS^T Q         (SS MMA: B = Q read MN-major)               -> TMEM [256+D,256+2D)
//   dQ^T = K^T dS^T       (SS MMA: A = K read MN-major, B = dS^T tile read MN-major; head dim 128)
//                          -> TMEM [128,256), over dP^T; lane = head-dim index.  A warpgroup of
//                             its own takes the whole tile into registers, hands the columns
//                             back, and adds the values to the fp32 accumulator with one
//                             reduction per query column: a warp's instruction covers 128
//                             contiguous bytes of a dQ row.
//                             (head dim 64 forms dQ = dS K instead; the compute warps reduce it.)
// Shared-memory bandwidth bounds this kernel: an SS MMA of 128 x 128 x 16 reads 8 KB of operands
// in the 64 cycles its arithmetic takes, which is all of the 128 bytes per cycle that shared
// memory delivers, so every other access on that data path (TMA writes of Q and dO, the dS^T
// stores, the loads of the per-row terms, global reductions) lengthens the MMAs.  That is why
// dQ leaves through registers and not through a shared-memory staging buffer as well.
// Head dim 128: warps 0-7 compute (two warpgroups split the 128 query columns), warps 8-11 drain
// dQ^T, warp 12 TMA producer, warp 13 MMA issuer, warps 14-15 idle (registers are re-divided
// between whole warpgroups).  Head dim 64: warps 0-7 compute, warp 8 producer, warp 9 MMA issuer.
// Grid: CTAs of a few (batch, head) pairs at a time, so that the Q / dO tiles and the dQ
// accumulator rows that the resident CTAs stream stay in L2.
#include <cstdio>
#include <cstring>

#include "host_util.h"
#include "tc_common.cuh"

namespace ra {

namespace {

using namespace ptx;

// 10 warps; with the drain warpgroup (head dim 128) 16
constexpr int bwd_threads(bool drain) { return drain ? 512 : 320; }
// Registers per thread after the re-division, with the drain warpgroup: every scheduler hosts two
// compute warps, one drain warp and one of the others, 2 * 152 + 152 + 56 = 512 = 16384 / 32.
constexpr int kRegsCompute = 152, kRegsDrain = 152, kRegsOther = 56;

template <int N>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr unsigned kProducerPollNs = 100;

struct BwdTcParams {
  CUtensorMap map_q, map_k, map_v, map_do;
  BwdParams p;
  const TileMeta* meta_q;
  const TileMeta* meta_kv;
  int n_q_tiles, n_kv_tiles;
  int group_heads;  // (batch, head) pairs whose CTAs are interleaved in the grid
  unsigned int* status;
};

enum Bar {
  KV_FULL = 0, Q_FULL0, Q_FULL1, Q_EMPTY0, Q_EMPTY1, DO_FULL0, DO_FULL1, DO_EMPTY0, DO_EMPTY1, S_FULL, DP_FULL, P_READY, DS_READY,
  DQ_FULL, DQ_DRAINED, DKDV_FULL, NUM_BARS
};

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

template <int D>
__global__ void __launch_bounds__(bwd_threads(D == 128), 1) tc_bwd_kernel(const __grid_constant__ BwdTcParams P) {
  constexpr bool DRAIN = D == 128;  // the drain warpgroup serves the dQ^T form
  constexpr int PRODUCER_WARP = DRAIN ? 12 : 8, MMA_WARP = PRODUCER_WARP + 1;
  constexpr int TILE_BYTES = kTileRows * D * 2;
  constexpr int PANELS = D / 64;
  constexpr int PANEL_BYTES = kTileRows * 128;
  constexpr int DS_BYTES = kTileRows * kTileRows * 2;
  constexpr int DO_ST = 2;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;          // 2 stages
  uint8_t* sdO = sQ + 2 * TILE_BYTES;     // DO_ST stages
  uint8_t* sdS = sdO + DO_ST * TILE_BYTES;  // [128 key rows][128 query cols] bf16, 2 panels, 128B swizzle
  float* sL = reinterpret_cast<float*>(sdS + DS_BYTES);  // [2][128]
  float* sDelta = sL + 2 * kTileRows;                     // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDelta + 2 * kTileRows);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const BwdParams& p = P.p;
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int bh_count = p.b * p.h;
  // groups of group_heads (batch, head) pairs; inside a group the pairs alternate and the K/V
  // tiles ascend (tile 0 has the most visible queries under a causal mask)
  const int per_group = P.group_heads * P.n_kv_tiles;
  const int grp = blockIdx.x / per_group, in_grp = blockIdx.x - grp * per_group;
  const int grp_n = min(P.group_heads, bh_count - grp * P.group_heads);
  const int bh = grp * P.group_heads + in_grp % grp_n;
  const int kt = in_grp / grp_n;
  const int hh = bh % p.h, bb = bh / p.h;
  const uint32_t kinds = p.mod.kinds;
  const bool masked = (kinds & kMetaKinds) != 0;  // the tile summaries are read
  const bool dense = (kinds & RA_MOD_DENSE) != 0;  // every tile takes the in-TMEM pass (it adds the bias tile)

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_BARS; ++i) {
      uint32_t cnt = (i == P_READY || i == DS_READY) ? 256u : (i == DQ_DRAINED) ? (DRAIN ? 128u : 256u) : 1u;
      mbar_init(&bars[i], cnt);
    }
    *abort_flag = (smem_u32(smem) & 1023u) ? 1u : 0u;  // the swizzled tiles need a 1024-byte aligned base
    if (*abort_flag) atomicOr(P.status, kStBwdProducer);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  TileMeta mk;
  if (masked) mk = P.meta_kv[bb * P.n_kv_tiles + kt];
  // First query tile >= i that has a pair visible to this CTA's K/V tile (n_q_tiles if there is
  // none), with kMixedBit set when that tile mixes visible and masked pairs and kContigBit when
  // its positions are contiguous.  All 32 lanes of a warp call it with the same i.  Each lane
  // classifies one tile of a window of 32 consecutive tiles and the window stays in registers:
  // the summaries are loaded once per 32 tiles, not once per tile (a load per tile put an L2
  // round trip on the critical path of every role), and a long masked stretch (the tiles before
  // the diagonal, other documents) costs one load per 32 tiles.
  constexpr int kMixedBit = 1 << 16, kContigBit = 1 << 17, kTileIdx = kMixedBit - 1;
  struct Window {
    int base = -(1 << 30);  // first tile of the window
    int cls = 0;            // this lane's tile: 0 skip, 1 all visible, 2 mixed; +4 contiguous positions
    int32_t pos0 = 0;       // first position of this lane's tile (valid when contiguous)
    int32_t hit_pos0 = 0;   // pos0 of the tile the last call returned
  };
  auto next_active = [&](Window& w, int i) -> int {
    if (!masked) return i < P.n_q_tiles ? (i | (dense ? kMixedBit : 0)) : P.n_q_tiles;
    while (i < P.n_q_tiles) {
      if (i < w.base || i >= w.base + 32) {
        w.base = i;
        w.cls = 0;
        const int t = i + lane;
        if (t < P.n_q_tiles) {
          const TileMeta mq = P.meta_q[bb * P.n_q_tiles + t];
          w.cls = classify_tiles(kinds, p.mod.window, mq, mk) | (mq.pos_contig ? 4 : 0);
          w.pos0 = mq.pos_min;
        }
      }
      const uint32_t vote = __ballot_sync(0xffffffffu, (w.cls & 3) != 0 && lane >= i - w.base);
      if (vote) {
        const int first = __ffs(vote) - 1;
        const int c = __shfl_sync(0xffffffffu, w.cls, first);
        w.hit_pos0 = __shfl_sync(0xffffffffu, w.pos0, first);
        return (w.base + first) | (((c & 3) == 2 || dense) ? kMixedBit : 0) | ((c & 4) ? kContigBit : 0);
      }
      i = w.base + 32;
    }
    return P.n_q_tiles;
  };

  // Every warp looks up the CTA's first visible query tile.  A K/V tile that no query of this
  // block sees (the tiles past the diagonal of a causal pair of shards) takes no tensor memory.
  Window win0;
  const int first_tile = next_active(win0, 0) & kTileIdx;
  const bool has_work = first_tile < P.n_q_tiles;
  if (warp == MMA_WARP && has_work) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = has_work ? __shfl_sync(0xffffffffu, *tmem_slot, 0) : 0u;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_dV = tmem_base + 256,
                 tmem_dK = tmem_base + 256 + D;
  const bool bad = *abort_flag != 0;

  if (bad) {
    // fall through to the common exit
  } else if (warp >= PRODUCER_WARP) {
    // the producer warp and the MMA warp; with the drain warpgroup they and two idle warps form
    // a warpgroup, which hands most of its registers to the others
    if constexpr (DRAIN) reg_dec<kRegsOther>();
    if (warp == PRODUCER_WARP) {
    // ------------------------------------------------------------ TMA producer
    // The whole warp walks the tile sequence (the scan is warp-wide); lane 0 polls and issues.
    if (lane == 0) {
      prefetch_tensormap(&P.map_q);
      prefetch_tensormap(&P.map_k);
      prefetch_tensormap(&P.map_v);
      prefetch_tensormap(&P.map_do);
    }
    Window wq = win0, wdo = win0;
    const int i = first_tile;
    if (i < P.n_q_tiles && lane == 0) {
      mbar_arrive_expect_tx(&bars[KV_FULL], 2 * TILE_BYTES);
      for (int pn = 0; pn < PANELS; ++pn) {
        tma_load_4d(sK + pn * PANEL_BYTES, &P.map_k, &bars[KV_FULL], pn * 64, hh, kt * kTileRows, bb);
        tma_load_4d(sV + pn * PANEL_BYTES, &P.map_v, &bars[KV_FULL], pn * 64, hh, kt * kTileRows, bb);
      }
    }
    // Two streams of loads: Q (with L and delta of its rows) and dO.  A Q stage is free after
    // dK of its tile, a dO stage already after dV of its tile, one MMA group earlier in the
    // next iteration: dO runs further ahead.  Both are polled so that neither blocks the other.
    const int64_t row_base = ((int64_t)bb * p.h + hh) * p.lq;
    int qi = i, doi = i, qn = 0, don = 0;
    long long t0 = 0;
    uint32_t idle = 0;
    while (qi < P.n_q_tiles || doi < P.n_q_tiles) {
      uint32_t ready = 0;
      if (lane == 0) {
        if (qi < P.n_q_tiles && mbar_test(&bars[Q_EMPTY0 + (qn & 1)], ((qn >> 1) & 1) ^ 1)) ready |= 1u;
        if (doi < P.n_q_tiles && mbar_test(&bars[DO_EMPTY0 + don % DO_ST], ((don / DO_ST) & 1) ^ 1)) ready |= 2u;
      }
      ready = __shfl_sync(0xffffffffu, ready, 0);
      if (ready & 1u) {
        if (lane == 0) {
          const int s = qn & 1;
          mbar_arrive_expect_tx(&bars[Q_FULL0 + s], TILE_BYTES + 2 * kTileRows * 4);
          for (int pn = 0; pn < PANELS; ++pn)
            tma_load_4d(sQ + s * TILE_BYTES + pn * PANEL_BYTES, &P.map_q, &bars[Q_FULL0 + s], pn * 64, hh, qi * kTileRows, bb);
          bulk_load(sL + s * kTileRows, p.row_nl2 + row_base + (int64_t)qi * kTileRows, kTileRows * 4, &bars[Q_FULL0 + s]);
          bulk_load(sDelta + s * kTileRows, p.row_nds + row_base + (int64_t)qi * kTileRows, kTileRows * 4, &bars[Q_FULL0 + s]);
        }
        qi = next_active(wq, qi + 1) & kTileIdx;
        ++qn;
      }
      if (ready & 2u) {
        if (lane == 0) {
          const int s = don % DO_ST;
          mbar_arrive_expect_tx(&bars[DO_FULL0 + s], TILE_BYTES);
          for (int pn = 0; pn < PANELS; ++pn)
            tma_load_4d(sdO + s * TILE_BYTES + pn * PANEL_BYTES, &P.map_do, &bars[DO_FULL0 + s], pn * 64, hh, doi * kTileRows, bb);
        }
        doi = next_active(wdo, doi + 1) & kTileIdx;
        ++don;
      }
      if (ready) {
        t0 = 0;
      } else {
        // every poll is a shared-memory access, and the MMAs need that bandwidth: poll about every 100 ns
        __nanosleep(kProducerPollNs);
      }
      if (!ready && (++idle & 63u) == 0) {  // bounded polling
        uint32_t stop = 0;
        if (lane == 0) {
          const long long now = clock64();
          if (t0 == 0) t0 = now;
          if (*abort_flag) {
            stop = 1;
          } else if (now - t0 > kWaitCycles) {
            *abort_flag = 1;
            atomicOr(P.status, kStBwdProducer);
            stop = 1;
          }
        }
        if (__shfl_sync(0xffffffffu, stop, 0)) break;
      }
    }
    } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------ MMA issuer
    {
      // every lane runs this loop; one elected lane issues each instruction
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);   // S^T, dP^T
      constexpr uint32_t idesc_dv = make_idesc_bf16(128, D, false, true);     // dV, dK: B MN-major
      // dQ: A and B MN-major.  D = 128 forms dQ^T (M = D, N = 128 queries); D = 64 forms dQ (M = 128 queries, N = D)
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, D == 128 ? 128 : D, true, true);
      // Low descriptor words: K-major views step 32 B per k-step inside a 64-column panel and one
      // panel (16 KB) per 4 k-steps; MN-major views step 16 rows (2 KB) per k-step, panels 16 KB apart.
      constexpr uint32_t kPanel16 = PANEL_BYTES >> 4, kStage16 = TILE_BYTES >> 4;
      const uint32_t k_km = desc_lo(smem_u32(sK), 16), k_mn = desc_lo(smem_u32(sK), PANEL_BYTES);
      const uint32_t v_km = desc_lo(smem_u32(sV), 16);
      const uint32_t q_km = desc_lo(smem_u32(sQ), 16), q_mn = desc_lo(smem_u32(sQ), PANEL_BYTES);
      const uint32_t do_km = desc_lo(smem_u32(sdO), 16), do_mn = desc_lo(smem_u32(sdO), PANEL_BYTES);
      const uint32_t ds_km = desc_lo(smem_u32(sdS), 16), ds_mn = desc_lo(smem_u32(sdS), PANEL_BYTES);
      auto km_off = [](int kk) -> uint32_t { return (kk >> 2) * kPanel16 + (kk & 3) * 2; };
      auto mn_off = [](int kk) -> uint32_t { return kk * (2048 >> 4); };
      auto issue_s = [&](int stage) {
        const uint32_t b0 = q_km + stage * kStage16;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss_warp(tmem_S, desc_from_lo(k_km + km_off(kk)), desc_from_lo(b0 + km_off(kk)), idesc_s, kk > 0);
        tc_commit_warp(&bars[S_FULL]);
      };
      auto issue_dp = [&](int stage) {
        const uint32_t b0 = do_km + stage * kStage16;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss_warp(tmem_dP, desc_from_lo(v_km + km_off(kk)), desc_from_lo(b0 + km_off(kk)), idesc_s, kk > 0);
        tc_commit_warp(&bars[DP_FULL]);
      };
      auto issue_dv = [&](int stage, bool first_tile) {
        const uint32_t b0 = do_mn + stage * kStage16;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t pcol = kk < 4 ? kk * 8 : 64 + (kk - 4) * 8;  // P^T columns of the two warpgroups
          mma_ts_warp(tmem_dV, tmem_S + pcol, desc_from_lo(b0 + mn_off(kk)), idesc_dv, (!first_tile) || kk > 0);
        }
      };
      // Issue order per query tile n (the tensor pipe executes in this order):
      //   S(n+1) | dQ(n) | dK(n) | dP(n+1) | dV(n+1)
      // so that the compute warps form P(n+1) under dQ(n)/dK(n), drain dQ(n) under dK(n), and
      // form dS(n+1) under dV(n+1)/S(n+2).
      bool ok = true;
      Window& win = win0;
      int i = first_tile;
      if (i < P.n_q_tiles) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bars[KV_FULL], 0, abort_flag, P.status, kStBwdMma) &&
                                         mbar_wait(&bars[Q_FULL0], 0, abort_flag, P.status, kStBwdMma) &&
                                         mbar_wait(&bars[DO_FULL0], 0, abort_flag, P.status, kStBwdMma));
        if (ok) {
          tc_fence_after();
          issue_s(0);
          issue_dp(0);
          ok = __all_sync(0xffffffffu, mbar_wait(&bars[P_READY], 0, abort_flag, P.status, kStBwdMma));
        }
        if (ok) {
          tc_fence_after();
          issue_dv(0, true);
          tc_commit_warp(&bars[DO_EMPTY0]);
        }
        for (int n = 0; ok; ++n) {
          const int s = n & 1, sn = (n + 1) & 1;
          const int dsn = (n + 1) % DO_ST;  // dO stage and phase of tile n + 1
          const uint32_t dphn = ((n + 1) / DO_ST) & 1;
          const uint32_t par = n & 1;
          const int inext = next_active(win, i + 1) & kTileIdx;
          const bool has_next = inext < P.n_q_tiles;
          if (has_next) {
            if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[Q_FULL0 + sn], ((n + 1) >> 1) & 1, abort_flag, P.status, kStBwdMma)))) break;
            tc_fence_after();
            issue_s(sn);
          }
          // dQ = dS K (into the dP^T columns), dK += dS^T Q
          if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[DS_READY], par, abort_flag, P.status, kStBwdMma)))) break;
          tc_fence_after();
          if constexpr (D == 128) {
            // dQ^T = K^T dS^T: lane = head-dim index, column = query, so that a warp's reduction
            // instruction covers 128 contiguous bytes of one dQ row
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              mma_ss_warp(tmem_dP, desc_from_lo(k_mn + mn_off(kk)), desc_from_lo(ds_mn + mn_off(kk)), idesc_dq, kk > 0);
          } else {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              mma_ss_warp(tmem_dP, desc_from_lo(ds_mn + mn_off(kk)), desc_from_lo(k_mn + mn_off(kk)), idesc_dq, kk > 0);
          }
          tc_commit_warp(&bars[DQ_FULL]);
          {
            const uint32_t b0 = q_mn + s * kStage16;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              mma_ss_warp(tmem_dK, desc_from_lo(ds_km + km_off(kk)), desc_from_lo(b0 + mn_off(kk)), idesc_dv,
                     (n > 0) || kk > 0);
          }
          tc_commit_warp(&bars[Q_EMPTY0 + s]);
          if (!has_next) break;
          if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[DQ_DRAINED], par, abort_flag, P.status, kStBwdMma)))) break;
          if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[DO_FULL0 + dsn], dphn, abort_flag, P.status, kStBwdMma)))) break;
          tc_fence_after();
          issue_dp(dsn);
          if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[P_READY], par ^ 1, abort_flag, P.status, kStBwdMma)))) break;
          tc_fence_after();
          issue_dv(dsn, false);
          tc_commit_warp(&bars[DO_EMPTY0 + dsn]);
          i = inext;
        }
        if (ok) tc_commit_warp(&bars[DKDV_FULL]);
      }
    }
    }
  } else if (DRAIN && warp >= 8) {
    // ------------------------------------------------------------ dQ^T drain (warps 8-11)
    if constexpr (DRAIN) {
      reg_inc<kRegsDrain>();
      // This thread owns head-dim index r of dQ^T; the 128 columns are the tile's queries.  The
      // whole tile goes to registers and the TMEM columns back to the MMA warp at once; then one
      // reduction per query: the warp's 32 lanes cover 128 contiguous bytes of that dQ row.
      const int r = (warp & 3) * 32 + lane;
      const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
      const int64_t qrow_base = ((int64_t)bb * p.h + hh) * p.lq;
      Window win = win0;
      bool ok = true;
      int i = first_tile;
      for (int n = 0; i < P.n_q_tiles; ++n) {
        if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[DQ_FULL], n & 1, abort_flag, P.status, kStBwdCompute)))) break;
        tc_fence_after();
        uint32_t dv[4][32];
#pragma unroll
        for (int j = 0; j < 4; ++j) tmem_ld32(tmem_dP + lane_off + 32 * j, dv[j]);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(&bars[DQ_DRAINED]);
        float* base = p.dq + (qrow_base + (int64_t)i * kTileRows) * 128 + r;
#pragma unroll
        for (int c = 0; c < 128; ++c)
          asm volatile("red.global.add.f32 [%0], %1;" ::"l"(base + c * 128), "f"(__uint_as_float(dv[c >> 5][c & 31])) : "memory");
        i = next_active(win, i + 1) & kTileIdx;
      }
    }
  } else {
    // ------------------------------------------------------------ compute (warps 0-7)
    if constexpr (DRAIN) reg_inc<kRegsCompute>();
    const int g = warp >> 2;                         // warpgroup: query columns [64g, 64g+64)
    const int r = (warp & 3) * 32 + lane;            // key row of this thread = TMEM lane
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const int kv_row = kt * kTileRows + r;
    const float scale2 = p.scale * kLog2e;
    const bool alibi = (kinds & RA_MOD_ALIBI) != 0;
    int32_t kpos = 0, kseg = 0;
    bool kpre = false;
    if (p.mod.kv_pos) kpos = p.mod.kv_pos[(int64_t)bb * p.lk + kv_row];
    if (p.mod.kv_seg) kseg = p.mod.kv_seg[(int64_t)bb * p.lk + kv_row];
    if (p.mod.kv_pre) kpre = p.mod.kv_pre[(int64_t)bb * p.lk + kv_row] != 0;
    const int64_t qrow_base = ((int64_t)bb * p.h + hh) * p.lq;
    bool ok = true;  // warp-uniform: the tile scan below votes across the warp
    float pf[64];        // P^T of the tile whose dS^T is formed next (this thread's row, 64 columns)
    uint32_t sv[2][32];
    const float alibi_over_scale = alibi ? p.mod.slopes[hh] / p.scale : 0.f;
    const float slope2 = alibi ? p.mod.slopes[hh] * kLog2e : 0.f;
    Window& win = win0;

    // One loop body serves every tile so that each phase exists once in the instruction
    // stream: step k does dS^T(k-1), then P^T(k), then the dQ drain of tile k-1.
    int i_prev = -1, e_cur = next_active(win, first_tile), i_cur = e_cur & kTileIdx;
    int32_t q0_cur = win.hit_pos0;  // first query position of the tile (used when its positions are contiguous)
    for (int k = 0; ok; ++k) {
      const bool have_prev = k > 0, have_cur = i_cur < P.n_q_tiles;
      if (!have_prev && !have_cur) break;
      const int e_next = have_cur ? next_active(win, i_cur + 1) : P.n_q_tiles;
      const int32_t q0_next = win.hit_pos0;
      if (have_prev) {
        // ---- dS^T = P^T * (dP^T * scale - delta * scale) of tile k-1 -> shared memory, 128-byte swizzle
        const int n = k - 1, s = n & 1;
        const float4* Dls = reinterpret_cast<const float4*>(sDelta + s * kTileRows + g * 64);
        if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[DP_FULL], n & 1, abort_flag, P.status, kStBwdCompute)))) break;
        tc_fence_after();
        tmem_ld32(tmem_dP + lane_off + g * 64, sv[0]);
        if constexpr (!DRAIN) tmem_ld32(tmem_dP + lane_off + g * 64 + 32, sv[1]);
        tc_wait_ld();
        // dS^T of the tile before may be overwritten now: dP^T of this tile was issued after the
        // MMAs that read it (dQ, dK), the tensor pipe runs in issue order, and DP_FULL's commit
        // covers everything issued before it
        uint8_t* row_ptr = sdS + g * PANEL_BYTES + r * 128;
        const uint64_t scl2 = pack2(p.scale, p.scale);
        // 8 query columns (one 16-byte chunk of this key row of dS^T) from 8 dP^T values
        auto ds_chunk = [&](int ch, const uint32_t* dp) {
          const float4 da = Dls[ch * 2], db = Dls[ch * 2 + 1];  // -delta * scale of 8 queries
          const uint64_t dl2[4] = {pack2(da.x, da.y), pack2(da.z, da.w), pack2(db.x, db.y), pack2(db.z, db.w)};
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = ch * 8 + e * 2;
            const uint64_t dp2 = pack2(__uint_as_float(dp[e * 2]), __uint_as_float(dp[e * 2 + 1]));
            float d0, d1;
            unpack2(mul2(pack2(pf[c], pf[c + 1]), fma2(dp2, scl2, dl2[e])), d0, d1);
            w[e] = pack_bf16(d0, d1);
          }
          *reinterpret_cast<uint4*>(row_ptr + ((ch ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        };
        if constexpr (DRAIN) {
          // fewer registers per thread here: the second 32 columns are loaded once half of the
          // first 32 (and the P^T values that went with them) are no longer needed
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) ds_chunk(ch, &sv[0][ch * 8]);
          tmem_ld32(tmem_dP + lane_off + g * 64 + 32, sv[1]);
#pragma unroll
          for (int ch = 2; ch < 4; ++ch) ds_chunk(ch, &sv[0][ch * 8]);
          tc_wait_ld();
#pragma unroll
          for (int ch = 4; ch < 8; ++ch) ds_chunk(ch, &sv[1][(ch - 4) * 8]);
        } else {
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) ds_chunk(ch, &sv[ch >> 2][(ch & 3) * 8]);
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&bars[DS_READY]);
      }
      if (have_cur) {
        // ---- P^T = exp2(S^T * scale2 - L * log2e) of tile k on this warpgroup's 64 query columns
        const int n = k, s = n & 1, i = i_cur;
        const bool need_mask = (e_cur & kMixedBit) != 0;
        // ALiBi over a tile of contiguous query positions with nothing masked is two FMAs per
        // score in registers; every other ALiBi tile takes the in-TMEM pass below
        const bool alibi_inline = alibi && !need_mask && (e_cur & kContigBit) != 0;
        if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[Q_FULL0 + s], (n >> 1) & 1, abort_flag, P.status, kStBwdCompute)))) break;
        const float4* Ls = reinterpret_cast<const float4*>(sL + s * kTileRows + g * 64);
        if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[S_FULL], n & 1, abort_flag, P.status, kStBwdCompute)))) break;
        tc_fence_after();
        if (need_mask || (alibi && !alibi_inline)) {  // tiles that mix visible and masked pairs, ALiBi over scattered positions
          const int64_t q0 = (int64_t)bb * p.lq + (int64_t)i * kTileRows + g * 64;
          fixup_scores_tmem<false>(tmem_S + lane_off + g * 64, 64, need_mask ? kinds : (kinds & RA_MOD_ALIBI),
                                   p.mod.window, alibi_over_scale, kpos, kseg, kpre,
                                   p.mod.q_pos ? p.mod.q_pos + q0 : nullptr, p.mod.q_seg ? p.mod.q_seg + q0 : nullptr,
                                   p.mod.q_pre ? p.mod.q_pre + q0 : nullptr, q0_cur + g * 64, (e_cur & kContigBit) != 0,
                                   dense ? p.mod.bias + (int64_t)bb * p.mod.bsb + (int64_t)hh * p.mod.bsh +
                                               ((int64_t)i * kTileRows + g * 64) * p.mod.bsq + kv_row
                                         : nullptr,
                                   p.mod.bsq, 1.f / p.scale);
        }
        tmem_ld32(tmem_S + lane_off + g * 64, sv[0]);
        tmem_ld32(tmem_S + lane_off + g * 64 + 32, sv[1]);
        tc_wait_ld();
        float sc = scale2;  // what is left to multiply the register values by
        if (alibi_inline) {
          // scale * s - slope * (q_pos - kv_pos), times log2(e), with q_pos = q0 + column; the
          // position differences are exact in fp32
          const float rr = slope2 * (float)(kpos - (q0_cur + g * 64));
#pragma unroll
          for (int c = 0; c < 64; ++c)
            sv[c >> 5][c & 31] = __float_as_uint(fmaf(-slope2, (float)c, fmaf(__uint_as_float(sv[c >> 5][c & 31]), scale2, rr)));
          sc = 1.f;
        }
        if (dense) {
          // With a dense bias tile the reference's arithmetic is kept as it is (ring.py:146): a row
          // whose L is -inf (it saw no key) gives exp(-inf + inf) = NaN.
#pragma unroll
          for (int c4 = 0; c4 < 16; ++c4) {
            const float4 lv = Ls[c4];
            const float l4[4] = {lv.x, lv.y, lv.z, lv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int c = c4 * 4 + e;
              pf[c] = ex2(fmaf(__uint_as_float(sv[c >> 5][c & 31]), sc, l4[e]));  // l4: -L * log2(e), unclamped
            }
          }
        } else {
          // A masked pair (-inf) gives exp2(-inf) = 0; the clamp in the row term keeps a row whose L
          // is -inf from turning that into exp2(-inf + inf).  Column pairs: packed arithmetic.
          const uint64_t sc2 = pack2(sc, sc);
#pragma unroll
          for (int c4 = 0; c4 < 16; ++c4) {
            const float4 lv = Ls[c4];
            const float l4[4] = {lv.x, lv.y, lv.z, lv.w};
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
              const int c = c4 * 4 + e;
              const uint64_t nl2 = pack2(l4[e], l4[e + 1]);  // min(-L * log2(e), 1e30) of the two queries
              const uint64_t x2 = fma2(pack2(__uint_as_float(sv[c >> 5][c & 31]), __uint_as_float(sv[(c + 1) >> 5][(c + 1) & 31])), sc2, nl2);
              float x0, x1;
              unpack2(x2, x0, x1);
              pf[c] = ex2(x0);
              pf[c + 1] = ex2(x1);
            }
          }
        }
        // P^T of warpgroup g: 32 packed columns at S column 64g, stored in two halves (fewer live registers)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = pack_bf16(pf[32 * hf + 2 * e], pf[32 * hf + 2 * e + 1]);
          tmem_st16(tmem_S + lane_off + g * 64 + 16 * hf, pk);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&bars[P_READY]);
      }
      if constexpr (!DRAIN) {
        if (have_prev) {
          // ---- dQ of tile k-1 (head dim 64): rows are queries; add this warpgroup's half of the columns
          const int n = k - 1;
          if (!(ok = __all_sync(0xffffffffu, mbar_wait(&bars[DQ_FULL], n & 1, abort_flag, P.status, kStBwdCompute)))) break;
          tc_fence_after();
          constexpr int HALF = D / 2;
          float* dq_row = p.dq + (qrow_base + (int64_t)i_prev * kTileRows + r) * D + g * HALF;
          tmem_ld32(tmem_dP + lane_off + g * HALF, sv[0]);
          tc_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            red_add_v4(dq_row + e, __uint_as_float(sv[0][e]), __uint_as_float(sv[0][e + 1]), __uint_as_float(sv[0][e + 2]),
                       __uint_as_float(sv[0][e + 3]));
          tc_fence_before();
          mbar_arrive(&bars[DQ_DRAINED]);
        }
      }
      if (!have_cur) break;
      i_prev = i_cur;
      e_cur = e_next;
      i_cur = e_cur & kTileIdx;
      q0_cur = q0_next;
    }
    const int n = (i_prev >= 0) ? 1 : 0;  // whether this CTA had any tile
    // ---- epilogue: dK, dV of this K/V tile
    if (ok && n > 0) ok = mbar_wait(&bars[DKDV_FULL], 0, abort_flag, P.status, kStBwdCompute);
    if (ok && n > 0) {
      tc_fence_after();
      constexpr int HALF = D / 2;
      const int64_t krow = ((int64_t)bb * p.h + hh) * p.lk + kv_row;
      float* dk_row = p.dk + krow * D + g * HALF;
      float* dv_row = p.dv + krow * D + g * HALF;
      const bool direct = p.dk_out.ptr != nullptr;  // ring of one: results go out in the input dtype
      const bool fresh = p.overwrite != 0;          // the fp32 buffers hold nothing yet: store, do not add
      __nv_bfloat16* dk_o = direct ? (__nv_bfloat16*)p.dk_out.ptr + (int64_t)bb * p.dk_out.sb +
                                         (int64_t)kv_row * p.dk_out.sl + (int64_t)hh * p.dk_out.sh + g * HALF
                                   : nullptr;
      __nv_bfloat16* dv_o = direct ? (__nv_bfloat16*)p.dv_out.ptr + (int64_t)bb * p.dv_out.sb +
                                         (int64_t)kv_row * p.dv_out.sl + (int64_t)hh * p.dv_out.sh + g * HALF
                                   : nullptr;
#pragma unroll 1
      for (int c = 0; c < HALF / 8; ++c) {
        uint32_t a[8];
        tmem_ld8(tmem_dK + lane_off + g * HALF + c * 8, a);
        tc_wait_ld();
        if (direct) {
          uint4 w;
          w.x = pack_bf16(__uint_as_float(a[0]), __uint_as_float(a[1]));
          w.y = pack_bf16(__uint_as_float(a[2]), __uint_as_float(a[3]));
          w.z = pack_bf16(__uint_as_float(a[4]), __uint_as_float(a[5]));
          w.w = pack_bf16(__uint_as_float(a[6]), __uint_as_float(a[7]));
          *reinterpret_cast<uint4*>(dk_o + c * 8) = w;
        } else {
#pragma unroll
          for (int e = 0; e < 8; e += 4) {
            float4 cur = fresh ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<float4*>(dk_row + c * 8 + e);
            cur.x += __uint_as_float(a[e]);
            cur.y += __uint_as_float(a[e + 1]);
            cur.z += __uint_as_float(a[e + 2]);
            cur.w += __uint_as_float(a[e + 3]);
            *reinterpret_cast<float4*>(dk_row + c * 8 + e) = cur;
          }
        }
        tmem_ld8(tmem_dV + lane_off + g * HALF + c * 8, a);
        tc_wait_ld();
        if (direct) {
          uint4 w;
          w.x = pack_bf16(__uint_as_float(a[0]), __uint_as_float(a[1]));
          w.y = pack_bf16(__uint_as_float(a[2]), __uint_as_float(a[3]));
          w.z = pack_bf16(__uint_as_float(a[4]), __uint_as_float(a[5]));
          w.w = pack_bf16(__uint_as_float(a[6]), __uint_as_float(a[7]));
          *reinterpret_cast<uint4*>(dv_o + c * 8) = w;
        } else {
#pragma unroll
          for (int e = 0; e < 8; e += 4) {
            float4 cur = fresh ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<float4*>(dv_row + c * 8 + e);
            cur.x += __uint_as_float(a[e]);
            cur.y += __uint_as_float(a[e + 1]);
            cur.z += __uint_as_float(a[e + 2]);
            cur.w += __uint_as_float(a[e + 3]);
            *reinterpret_cast<float4*>(dv_row + c * 8 + e) = cur;
          }
        }
      }
    } else if (ok && n == 0 && p.dk_out.ptr != nullptr) {
      // no query tile sees this K/V tile: its gradients are zero, and in direct mode nobody else writes them
      constexpr int HALF = D / 2;
      __nv_bfloat16* dk_o = (__nv_bfloat16*)p.dk_out.ptr + (int64_t)bb * p.dk_out.sb + (int64_t)kv_row * p.dk_out.sl +
                            (int64_t)hh * p.dk_out.sh + g * HALF;
      __nv_bfloat16* dv_o = (__nv_bfloat16*)p.dv_out.ptr + (int64_t)bb * p.dv_out.sb + (int64_t)kv_row * p.dv_out.sl +
                            (int64_t)hh * p.dv_out.sh + g * HALF;
#pragma unroll 1
      for (int c = 0; c < HALF / 8; ++c) {
        *reinterpret_cast<uint4*>(dk_o + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(dv_o + c * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    else if (ok && n == 0 && p.overwrite) {
      // no query tile sees this K/V tile and the fp32 buffers were not cleared: its rows are zero
      constexpr int HALF = D / 2;
      const int64_t krow = ((int64_t)bb * p.h + hh) * p.lk + kv_row;
      float4* dk_row = reinterpret_cast<float4*>(p.dk + krow * D + g * HALF);
      float4* dv_row = reinterpret_cast<float4*>(p.dv + krow * D + g * HALF);
#pragma unroll 1
      for (int c = 0; c < HALF / 4; ++c) dk_row[c] = dv_row[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP && has_work) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D>
cudaError_t launch_bwd(const BwdTcParams& P, cudaStream_t s) {
  constexpr size_t kSmem = 6 * kTileRows * D * 2 + kTileRows * kTileRows * 2 + 4 * kTileRows * 4 + NUM_BARS * 8 + 64;
  constexpr size_t kRequest = kSmem < 120 * 1024 ? 120 * 1024 : kSmem;  // one CTA per SM: it owns all of TMEM
  auto kern = tc_bwd_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRequest);
  if (e != cudaSuccess) return e;
  kern<<<P.n_kv_tiles * P.p.b * P.p.h, bwd_threads(D == 128), kRequest, s>>>(P);
  count_launch();
  return cudaGetLastError();
}

bool aligned16(const TensorView& t) {
  return (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 && (t.sb % 8) == 0 && (t.sl % 8) == 0 && (t.sh % 8) == 0;
}

}  // namespace

const char* tc_bwd_unsupported_reason(const BwdParams& p, int dtype) {
  if (dtype != RA_DTYPE_BF16) return "inputs are not bf16";
  if (p.dk_dim != p.dv_dim || (p.dk_dim != 64 && p.dk_dim != 128)) return "head dims must be equal and 64 or 128";
  if (p.lq % kTileRows || p.lk % kTileRows) return "lq and lk must be multiples of 128";
  if (p.lq / kTileRows > kMaxTiles || p.lk / kTileRows > kMaxTiles) return "more than 4096 tiles along one axis";
  if ((p.mod.kinds & RA_MOD_DENSE) && ((p.mod.bsb % 4) || (p.mod.bsh % 4) || (p.mod.bsq % 4) ||
                                       (reinterpret_cast<uintptr_t>(p.mod.bias) & 15)))
    return "the dense bias needs a 16-byte aligned base and strides that are multiples of 4 floats";
  if (!aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.dout))
    return "q/k/v/dout need 16-byte aligned base and strides";
  if ((reinterpret_cast<uintptr_t>(p.lse) & 15) || (reinterpret_cast<uintptr_t>(p.delta) & 15) ||
      (reinterpret_cast<uintptr_t>(p.dq) & 15) || (reinterpret_cast<uintptr_t>(p.dk) & 15) ||
      (reinterpret_cast<uintptr_t>(p.dv) & 15))
    return "lse/delta/dq/dk/dv need 16-byte aligned bases";
  if (!(p.scale > 0.f)) return "sm_scale must be positive";
  if (p.dk_out.ptr && (!aligned16(p.dk_out) || !p.dv_out.ptr || !aligned16(p.dv_out)))
    return "dk/dv results need 16-byte aligned bases and strides";
  return nullptr;
}

cudaError_t tc_bwd_block(const BwdParams& p, cudaStream_t s) {
  BwdTcParams P;
  memset(&P, 0, sizeof(P));
  P.p = p;
  P.n_q_tiles = p.lq / kTileRows;
  P.n_kv_tiles = p.lk / kTileRows;
  const char* why = nullptr;
  if (!make_tile_map(&P.map_q, p.q, p.b, p.lq, p.h, p.dk_dim, kTileRows, &why) ||
      !make_tile_map(&P.map_k, p.k, p.b, p.lk, p.h, p.dk_dim, kTileRows, &why) ||
      !make_tile_map(&P.map_v, p.v, p.b, p.lk, p.h, p.dv_dim, kTileRows, &why) ||
      !make_tile_map(&P.map_do, p.dout, p.b, p.lq, p.h, p.dv_dim, kTileRows, &why))
    return cudaErrorNotSupported;
  P.status = device_status_word();
  if (!P.status) return cudaErrorInvalidSymbol;
  // CTAs that are resident together should stream the same Q / dO tiles and add into the same
  // dQ rows: interleave only as many (batch, head) pairs as keep those within about 64 MB of L2
  const int64_t per_head = (int64_t)p.lq * p.dk_dim * (2 + 2 + 4);
  int64_t group = (64ll << 20) / (per_head > 0 ? per_head : 1);
  if (group < 1) group = 1;
  if (group > (int64_t)p.b * p.h) group = (int64_t)p.b * p.h;
  P.group_heads = (int)group;
  TileMeta* meta = nullptr;
  float* terms = nullptr;
  cudaError_t e = cudaSuccess;
  if (!p.row_nl2 || !p.row_nds) {  // block-level callers pass L and delta as the reference does
    const int64_t rows = (int64_t)p.b * p.h * p.lq;
    const size_t each = ((size_t)rows * sizeof(float) + 255) / 256 * 256;
    if ((e = scratch_alloc((void**)&terms, 2 * each, s)) != cudaSuccess) return e;
    float* nl2 = terms;
    float* nds = reinterpret_cast<float*>(reinterpret_cast<char*>(terms) + each);
    e = launch_bwd_row_terms(p.lse, p.delta, p.scale, (p.mod.kinds & RA_MOD_DENSE) ? 0 : 1, rows, nl2, nds, s);
    P.p.row_nl2 = nl2;
    P.p.row_nds = nds;
  }
  if (e == cudaSuccess && (p.mod.kinds & kMetaKinds)) {
    const size_t n = (size_t)p.b * (P.n_q_tiles + P.n_kv_tiles);
    if ((e = scratch_alloc((void**)&meta, n * sizeof(TileMeta), s)) != cudaSuccess) {
      if (terms) cudaFreeAsync(terms, s);
      return e;
    }
    TileMeta* mq = meta;
    TileMeta* mk = meta + (size_t)p.b * P.n_q_tiles;
    if ((e = launch_tile_meta(mq, p.mod.q_pos, p.mod.q_seg, p.mod.q_pre, p.b, p.lq, s)) == cudaSuccess)
      e = launch_tile_meta(mk, p.mod.kv_pos, p.mod.kv_seg, p.mod.kv_pre, p.b, p.lk, s);
    P.meta_q = mq;
    P.meta_kv = mk;
  }
  if (e == cudaSuccess) e = p.dk_dim == 128 ? launch_bwd<128>(P, s) : launch_bwd<64>(P, s);
  if (meta) cudaFreeAsync(meta, s);  // stream-ordered: after the kernels above, also when one failed to launch
  if (terms) cudaFreeAsync(terms, s);
  return e;
}

}  // namespace ra

