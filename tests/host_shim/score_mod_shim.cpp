// Host build of the score-mod rules (csrc/score_mod.h) for tests/test_score_mod_host.py:
// the per-pair rule and the tile classification exactly as the kernels compile them.
#include "score_mod.h"

extern "C" {

// meta: pos_min, pos_max, seg_min, seg_max, pre_any, pre_all, pos_contig
int ra_host_classify(uint32_t kinds, int32_t window, const int32_t* q, const int32_t* k) {
  ra::TileMeta mq{q[0], q[1], q[2], q[3], q[4], q[5], q[6], 0};
  ra::TileMeta mk{k[0], k[1], k[2], k[3], k[4], k[5], k[6], 0};
  return ra::classify_tiles(kinds, window, mq, mk);
}

// Number of visible pairs between nq query tokens and nk key tokens under the per-pair rule.
int64_t ra_host_count_visible(uint32_t kinds, int32_t window, int nq, const int32_t* qpos, const int32_t* qseg,
                              const uint8_t* qpre, int nk, const int32_t* kpos, const int32_t* kseg,
                              const uint8_t* kpre) {
  int64_t n = 0;
  for (int i = 0; i < nq; ++i)
    for (int j = 0; j < nk; ++j)
      n += ra::apply_mod(0.f, kinds, window, 0.f, qpos[i], qseg[i], qpre[i] != 0, kpos[j], kseg[j], kpre[j] != 0) == 0.f;
  return n;
}

// The per-pair rule on its own: 1 visible, 0 masked; *score gets the modified score.
int ra_host_apply_mod(float s, uint32_t kinds, int32_t window, float slope, int32_t qpos, int32_t qseg, int qpre,
                      int32_t kpos, int32_t kseg, int kpre, float* score) {
  const float y = ra::apply_mod(s, kinds, window, slope, qpos, qseg, qpre != 0, kpos, kseg, kpre != 0);
  *score = y;
  return y == -INFINITY ? 0 : 1;
}
}
