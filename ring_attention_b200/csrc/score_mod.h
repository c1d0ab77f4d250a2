// The score-mod rules shared by every kernel and by the ring plan: whether one (query, key)
// pair is visible, and what the 128-token summaries of a query tile and a key tile say about
// all of their pairs.  Plain C++ that also compiles for the host, so that the rules can be
// checked against each other exhaustively without a GPU (tests/test_score_mod_host.py).
#pragma once
#include <math.h>
#include <stdint.h>

#include "ring_attention_b200.h"

#if defined(__CUDACC__)
#define RA_HD __host__ __device__ __forceinline__
#else
#define RA_HD inline
#endif

namespace ra {

// One (query, key) score after scaling: mask + bias exactly as the reference's bias_fn
// variants would produce it (ring.py:386-408), -inf where the pair is masked.
RA_HD float apply_mod(float s, uint32_t kinds, int32_t window, float slope, int32_t qpos, int32_t qseg, bool qpre,
                      int32_t kpos, int32_t kseg, bool kpre) {
  bool vis = true;
  if (kinds & RA_MOD_SEGMENT) vis = vis && (qseg == kseg);
  if (kinds & RA_MOD_CAUSAL) {
    vis = vis && (kpos <= qpos);
  } else if (kinds & RA_MOD_PREFIX) {
    vis = vis && ((qpre && kpre) || (kpos <= qpos));
  }
  if (kinds & RA_MOD_WINDOW) vis = vis && ((qpos - kpos) < window);
  if (kinds & RA_MOD_ALIBI) s -= slope * (float)(qpos - kpos);
  return vis ? s : -INFINITY;
}

// Range summary of the per-token score-mod arrays over one 128-token tile.
struct TileMeta {
  int32_t pos_min, pos_max, seg_min, seg_max;
  int32_t pre_any, pre_all;
  int32_t pos_contig;  // 1 when the tile's positions are pos[0], pos[0] + 1, ... (then pos[0] == pos_min)
  int32_t pad1;
};

// 0: every pair of the tile pair is masked; 1: every pair is visible; 2: mixed (or unknown:
// 2 is always a safe answer, 0 and 1 are promises).
RA_HD int classify_tiles(uint32_t kinds, int32_t window, const TileMeta& q, const TileMeta& k) {
  bool skip = false, full = true;
  if (kinds & RA_MOD_SEGMENT) {
    if (q.seg_max < k.seg_min || k.seg_max < q.seg_min) skip = true;
    if (!(q.seg_min == q.seg_max && k.seg_min == k.seg_max && q.seg_min == k.seg_min)) full = false;
  }
  const bool causal_none = k.pos_min > q.pos_max, causal_all = k.pos_max <= q.pos_min;
  if (kinds & RA_MOD_CAUSAL) {
    if (causal_none) skip = true;
    if (!causal_all) full = false;
  } else if (kinds & RA_MOD_PREFIX) {
    const bool pre_none = !(q.pre_any && k.pre_any), pre_all = q.pre_all && k.pre_all;
    if (causal_none && pre_none) skip = true;
    if (!(causal_all || pre_all)) full = false;
  }
  if (kinds & RA_MOD_WINDOW) {
    if ((long long)q.pos_min - (long long)k.pos_max >= (long long)window) skip = true;
    if (!((long long)q.pos_max - (long long)k.pos_min < (long long)window)) full = false;
  }
  return skip ? 0 : (full ? 1 : 2);
}

}  // namespace ra
