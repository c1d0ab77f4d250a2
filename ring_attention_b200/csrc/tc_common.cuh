// Pieces shared by the tcgen05 forward and backward block kernels: per-tile mask
// metadata, tile classification, TMA descriptor construction, the device status word.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace ra {

constexpr int kTileRows = 128;     // rows of one q tile / one kv tile
constexpr int kMaxTiles = 4096;    // most tiles one block (shard) may have along either axis

constexpr uint32_t kMaskKinds = RA_MOD_CAUSAL | RA_MOD_SEGMENT | RA_MOD_PREFIX | RA_MOD_WINDOW;
// Score-mods that read the tile summaries (ALiBi reads pos_contig to choose its in-loop form).
constexpr uint32_t kMetaKinds = kMaskKinds | RA_MOD_ALIBI;

// Applies the score-mod to raw (unscaled) scores that sit in TMEM, in place: this thread's
// TMEM lane, `ncols` columns (a multiple of 16) from `taddr`.  Masked pairs become -inf and the
// ALiBi bias is added divided by the softmax scale, so that the kernels' main loops, which
// multiply by the scale, see exactly scale * s + bias.  Only tiles that mix visible and masked
// pairs (or ALiBi tiles over scattered positions) come here; it is a rolled loop on purpose: the
// main loops stay free of mask code and small enough for the instruction cache.  The next 16
// columns are in flight while the current 16 are worked on.  When the columns' positions are
// contiguous (`col_contig`: position of column c is col_pos0 + c) they are not loaded.
// kRowIsQuery: the thread's row is a query and columns are keys (forward); else the thread's
// row is a key and columns are queries (backward, transposed tiles).
// A dense bias tile (RA_MOD_DENSE: the materialised bias_fn result of ring.py:60-61) is added
// here as well, divided by the scale like the ALiBi term: `bias` points at this thread's row
// and the tile's first column, consecutive columns are `bias_col_stride` floats apart (1 in the
// forward, where a thread reads 64 contiguous bytes per 16 columns; the bias row stride in the
// backward, where the lanes of a warp read consecutive floats of one bias row).
template <bool kRowIsQuery>
__device__ __noinline__ void fixup_scores_tmem(uint32_t taddr, int ncols, uint32_t kinds, int32_t window,
                                               float alibi_over_scale, int32_t row_pos, int32_t row_seg,
                                               bool row_pre, const int32_t* col_pos, const int32_t* col_seg,
                                               const uint8_t* col_pre, int32_t col_pos0, bool col_contig,
                                               const float* bias = nullptr, int64_t bias_col_stride = 1,
                                               float inv_scale = 0.f) {
  uint32_t cur[16], nxt[16];
  ptx::tmem_ld16(taddr, cur);
#pragma unroll 1
  for (int c0 = 0; c0 < ncols; c0 += 16) {
    ptx::tc_wait_ld();
    const bool more = c0 + 16 < ncols;
    if (more) ptx::tmem_ld16(taddr + c0 + 16, nxt);
    if (bias) {
      float bv[16];
      if constexpr (kRowIsQuery) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias + c0) + j);
          bv[4 * j] = b4.x, bv[4 * j + 1] = b4.y, bv[4 * j + 2] = b4.z, bv[4 * j + 3] = b4.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) bv[e] = __ldg(bias + (int64_t)(c0 + e) * bias_col_stride);
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) cur[e] = __float_as_uint(fmaf(bv[e], inv_scale, __uint_as_float(cur[e])));
    }
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const int32_t cpos = col_contig ? col_pos0 + c0 + e : (col_pos ? __ldg(col_pos + c0 + e) : 0);
      const int32_t cseg = col_seg ? __ldg(col_seg + c0 + e) : 0;
      const bool cpre = col_pre ? (__ldg(col_pre + c0 + e) != 0) : false;
      const float x = __uint_as_float(cur[e]);
      const float y = kRowIsQuery
                          ? apply_mod(x, kinds, window, alibi_over_scale, row_pos, row_seg, row_pre, cpos, cseg, cpre)
                          : apply_mod(x, kinds, window, alibi_over_scale, cpos, cseg, cpre, row_pos, row_seg, row_pre);
      cur[e] = __float_as_uint(y);
    }
    ptx::tmem_st16(taddr + c0, cur);
    if (more) {
      ptx::tc_wait_ld();
#pragma unroll
      for (int e = 0; e < 16; ++e) cur[e] = nxt[e];
    }
  }
  ptx::tc_wait_st();
}

// Host side -----------------------------------------------------------------------------
// Tensor map over a [b, len, h, d] bf16 tensor with box {64 elements of d, 1 head, 128 rows,
// 1 batch} and the 128-byte swizzle the UMMA descriptors expect.  Returns false (with a
// reason) when the driver refuses the layout.
bool make_tile_map(CUtensorMap* map, const TensorView& t, int b, int len, int h, int d, int box_rows,
                   const char** why);

// Launches the kernel that fills TileMeta[b][n_tiles] for one side (q or kv).
cudaError_t launch_tile_meta(TileMeta* out, const int32_t* pos, const int32_t* seg, const uint8_t* pre,
                             int b, int len, cudaStream_t s);

// Stream-ordered scratch (tile summaries) from a memory pool of this library, one per device,
// that keeps what it has been given: the default pool hands unused memory back to the driver at
// every synchronisation, and the next call's allocation then costs milliseconds on the stream.
// Free with cudaFreeAsync on the same stream.
cudaError_t scratch_alloc(void** ptr, size_t bytes, cudaStream_t s);

// Device status word of the current device (bit set = a bounded wait ran out).
unsigned int* device_status_word();

// Failure codes OR-ed into the status word.
constexpr uint32_t kStFwdProducer = 1u << 0, kStFwdMma = 1u << 1, kStFwdSoftmax = 1u << 2;
constexpr uint32_t kStBwdProducer = 1u << 8, kStBwdMma = 1u << 9, kStBwdCompute = 1u << 10;

}  // namespace ra
