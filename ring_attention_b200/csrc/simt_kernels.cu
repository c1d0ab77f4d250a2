// fp32 CUDA-core block kernels: any shape (ragged tiles, head dims 1..256, cross
// attention), any score-mod including a dense bias tile, fp32 or bf16 inputs with all
// arithmetic in fp32.  They are the exact path (1e-5 against an fp64 restatement of
// ring_attention/ring.py:58-76 and :140-157) and serve every shape the tcgen05 kernels
// do not take.
#include <math.h>

#include "common.cuh"

namespace ra {

namespace {

constexpr int BM = 64;   // query rows per tile
constexpr int BN = 64;   // key rows per tile
constexpr int DC = 32;   // head-dim chunk staged for the QK^T / dO V^T products
constexpr int LDS = 33;  // padded row pitch of the staged chunks
constexpr int LDP = 65;  // padded row pitch of the P / dS tiles
constexpr int NT = 256;  // threads per block: 16 x 16, thread (ty,tx) owns rows 4ty..4ty+3

__device__ __forceinline__ float half_warp_max(float x) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float half_warp_sum(float x) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// Stage a [64 x 32] chunk of a [rows x dim] operand (rows from row0, columns from c0),
// zero filled outside the tensor.
template <typename T>
__device__ __forceinline__ void stage_chunk(float* dst, const T* base, int64_t sl, int row0,
                                            int nrows, int c0, int dim, int tid) {
  for (int e = tid; e < 64 * DC; e += NT) {
    int r = e >> 5, c = e & 31;
    float x = 0.f;
    if (row0 + r < nrows && c0 + c < dim) x = load_as_float(base + (int64_t)(row0 + r) * sl + c0 + c);
    dst[r * LDS + c] = x;
  }
}

// acc[i][j] += sum_c A[4ty+i][c] * B[tx+16j][c] over one staged chunk.
__device__ __forceinline__ void mma_chunk(float (&acc)[4][4], const float* As, const float* Bs,
                                          int ty, int tx) {
#pragma unroll 8
  for (int kk = 0; kk < DC; ++kk) {
    float a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = As[(ty * 4 + i) * LDS + kk];
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = Bs[(tx + 16 * j) * LDS + kk];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

struct ModTile {
  int32_t qpos[4], qseg[4], kpos[4], kseg[4];
  bool qpre[4], kpre[4];
  float slope;
};

__device__ __forceinline__ void load_mod_rows(ModTile& t, const ModParams& mod, int bb, int hh,
                                              int lq, int q0, int ty) {
  t.slope = (mod.kinds & RA_MOD_ALIBI) ? mod.slopes[hh] : 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int row = q0 + ty * 4 + i;
    bool ok = row < lq;
    int64_t idx = (int64_t)bb * lq + row;
    t.qpos[i] = (mod.q_pos && ok) ? mod.q_pos[idx] : 0;
    t.qseg[i] = (mod.q_seg && ok) ? mod.q_seg[idx] : 0;
    t.qpre[i] = (mod.q_pre && ok) ? (mod.q_pre[idx] != 0) : false;
  }
}
__device__ __forceinline__ void load_mod_cols(ModTile& t, const ModParams& mod, int bb, int lk,
                                              int k0, int tx) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int col = k0 + tx + 16 * j;
    bool ok = col < lk;
    int64_t idx = (int64_t)bb * lk + col;
    t.kpos[j] = (mod.kv_pos && ok) ? mod.kv_pos[idx] : 0;
    t.kseg[j] = (mod.kv_seg && ok) ? mod.kv_seg[idx] : 0;
    t.kpre[j] = (mod.kv_pre && ok) ? (mod.kv_pre[idx] != 0) : false;
  }
}

// True when no (row, column) pair of this thread's 4x4 patch is visible under the mask
// kinds (bias values do not matter here).  Used to skip tiles that are fully masked.
__device__ __forceinline__ bool patch_all_masked(const ModTile& t, const ModParams& mod, int q0,
                                                 int k0, int lq, int lk, int ty, int tx) {
  const uint32_t mask_kinds = mod.kinds & (RA_MOD_CAUSAL | RA_MOD_SEGMENT | RA_MOD_PREFIX | RA_MOD_WINDOW);
  bool any = false;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      bool in = (q0 + ty * 4 + i < lq) && (k0 + tx + 16 * j < lk);
      float x = apply_mod(0.f, mask_kinds, mod.window, 0.f, t.qpos[i], t.qseg[i], t.qpre[i], t.kpos[j],
                          t.kseg[j], t.kpre[j]);
      any = any || (in && x == 0.f);
    }
  return !any;
}

// scores = acc * scale, then mask / bias.  Columns past lk become -inf.
__device__ __forceinline__ void score_tile(float (&s)[4][4], const ModTile& t, const ModParams& mod,
                                           float scale, int bb, int hh, int q0, int k0, int lq,
                                           int lk, int ty, int tx) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int row = q0 + ty * 4 + i;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int col = k0 + tx + 16 * j;
      float x = s[i][j] * scale;
      if ((mod.kinds & RA_MOD_DENSE) && row < lq && col < lk)
        x += mod.bias[(int64_t)bb * mod.bsb + (int64_t)hh * mod.bsh + (int64_t)row * mod.bsq + col];
      x = apply_mod(x, mod.kinds, mod.window, t.slope, t.qpos[i], t.qseg[i], t.qpre[i], t.kpos[j],
                    t.kseg[j], t.kpre[j]);
      s[i][j] = (col < lk) ? x : -INFINITY;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Forward block: one online-softmax update of (o, m, l) with one K/V block
// (ring.py:58-76; ring_kernel.py:41-120).
// ---------------------------------------------------------------------------------------
template <typename T, int D_PAD>
__global__ void __launch_bounds__(NT) simt_fwd_kernel(const FwdParams p) {
  extern __shared__ float smem[];
  float* Qs = smem;
  float* Ks = Qs + 64 * LDS;
  float* Ps = Ks + 64 * LDS;
  float* Vs = Ps + 64 * LDP;  // [64][D_PAD]
  constexpr int NJ = D_PAD / 16;

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int q0 = blockIdx.x * BM, hh = blockIdx.y, bb = blockIdx.z;
  const T* qb = (const T*)p.q.ptr + (int64_t)bb * p.q.sb + (int64_t)hh * p.q.sh;
  const T* kb = (const T*)p.k.ptr + (int64_t)bb * p.k.sb + (int64_t)hh * p.k.sh;
  const T* vb = (const T*)p.v.ptr + (int64_t)bb * p.v.sb + (int64_t)hh * p.v.sh;
  const int64_t row_base = ((int64_t)bb * p.h + hh) * p.lq;

  float m_run[4], l_run[4], o_acc[4][NJ];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int row = q0 + ty * 4 + i;
    bool ld = (!p.first) && row < p.lq;
    m_run[i] = ld ? p.m[row_base + row] : -INFINITY;
    l_run[i] = ld ? p.l[row_base + row] : 0.f;
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) {
      int c = tx + 16 * jj;
      o_acc[i][jj] = (ld && c < p.dv) ? p.o[(row_base + row) * p.dv + c] : 0.f;
    }
  }
  ModTile mt;
  load_mod_rows(mt, p.mod, bb, hh, p.lq, q0, ty);

  const bool can_skip = (p.mod.kinds & (RA_MOD_CAUSAL | RA_MOD_SEGMENT | RA_MOD_PREFIX | RA_MOD_WINDOW)) != 0;
  for (int k0 = 0; k0 < p.lk; k0 += BN) {
    load_mod_cols(mt, p.mod, bb, p.lk, k0, tx);
    // A fully masked tile leaves (o, m, l) unchanged (p = 0, correction = 1): skip it.
    if (can_skip && !__syncthreads_or(!patch_all_masked(mt, p.mod, q0, k0, p.lq, p.lk, ty, tx))) continue;
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    for (int dc = 0; dc < p.dk; dc += DC) {
      stage_chunk(Qs, qb, p.q.sl, q0, p.lq, dc, p.dk, tid);
      stage_chunk(Ks, kb, p.k.sl, k0, p.lk, dc, p.dk, tid);
      __syncthreads();
      mma_chunk(s, Qs, Ks, ty, tx);
      __syncthreads();
    }
    for (int e = tid; e < 64 * D_PAD; e += NT) {
      int r = e / D_PAD, c = e % D_PAD;
      float x = 0.f;
      if (k0 + r < p.lk && c < p.dv) x = load_as_float(vb + (int64_t)(k0 + r) * p.v.sl + c);
      Vs[e] = x;
    }
    score_tile(s, mt, p.mod, p.scale, bb, hh, q0, k0, p.lq, p.lk, ty, tx);

#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float mx = fmaxf(fmaxf(s[i][0], s[i][1]), fmaxf(s[i][2], s[i][3]));
      mx = half_warp_max(mx);
      float m_new = fmaxf(m_run[i], mx);                                   // ring.py:63
      float corr = (m_new == -INFINITY) ? 0.f : expf(m_run[i] - m_new);    // ring.py:65-66
      float rs = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float pe = (m_new == -INFINITY) ? 0.f : expf(s[i][j] - m_new);     // ring.py:68-69
        rs += pe;
        Ps[(ty * 4 + i) * LDP + tx + 16 * j] = pe;
      }
      rs = half_warp_sum(rs);
      l_run[i] = corr * l_run[i] + rs;                                     // ring.py:75
      m_run[i] = m_new;
#pragma unroll
      for (int jj = 0; jj < NJ; ++jj) o_acc[i][jj] *= corr;                // ring.py:72
    }
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < BN; ++kk) {
      float pr[4], vv[NJ];
#pragma unroll
      for (int i = 0; i < 4; ++i) pr[i] = Ps[(ty * 4 + i) * LDP + kk];
#pragma unroll
      for (int jj = 0; jj < NJ; ++jj) vv[jj] = Vs[kk * D_PAD + tx + 16 * jj];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) o_acc[i][jj] = fmaf(pr[i], vv[jj], o_acc[i][jj]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int row = q0 + ty * 4 + i;
    if (row >= p.lq) continue;
    if (tx == 0) {
      p.m[row_base + row] = m_run[i];
      p.l[row_base + row] = l_run[i];
    }
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) {
      int c = tx + 16 * jj;
      if (c < p.dv) p.o[(row_base + row) * p.dv + c] = o_acc[i][jj];
    }
  }
}

// ---------------------------------------------------------------------------------------
// Backward block (ring.py:140-157; ring_kernel.py:303-384): one block of keys per CTA,
// loop over query tiles; dK/dV in registers, dQ through fp32 atomics.
// ---------------------------------------------------------------------------------------
template <typename T, int D_PAD>
__global__ void __launch_bounds__(NT) simt_bwd_kernel(const BwdParams p) {
  extern __shared__ float smem[];
  float* As = smem;             // [64][LDS]
  float* Bs = As + 64 * LDS;    // [64][LDS]
  float* Ps = Bs + 64 * LDS;    // [64 q][LDP]
  float* Ds = Ps + 64 * LDP;    // [64 q][LDP]  dS
  float* Ts = Ds + 64 * LDP;    // [64][64] operand tile for the second-stage products
  constexpr int NJ = D_PAD / 16;
  constexpr int NCH = D_PAD / 64 > 0 ? D_PAD / 64 : 1;  // 64-column chunks
  constexpr int JPC = NJ / NCH;                          // accumulator columns per chunk

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int k0 = blockIdx.x * BN, hh = blockIdx.y, bb = blockIdx.z;
  const T* qb = (const T*)p.q.ptr + (int64_t)bb * p.q.sb + (int64_t)hh * p.q.sh;
  const T* kb = (const T*)p.k.ptr + (int64_t)bb * p.k.sb + (int64_t)hh * p.k.sh;
  const T* vb = (const T*)p.v.ptr + (int64_t)bb * p.v.sb + (int64_t)hh * p.v.sh;
  const T* dob = (const T*)p.dout.ptr + (int64_t)bb * p.dout.sb + (int64_t)hh * p.dout.sh;
  const int64_t qrow_base = ((int64_t)bb * p.h + hh) * p.lq;
  const int64_t krow_base = ((int64_t)bb * p.h + hh) * p.lk;

  float dk_acc[4][NJ], dv_acc[4][NJ];  // rows = keys 4ty+i, cols tx+16jj
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) dk_acc[i][jj] = dv_acc[i][jj] = 0.f;

  ModTile mt;
  load_mod_cols(mt, p.mod, bb, p.lk, k0, tx);

  const bool can_skip = (p.mod.kinds & (RA_MOD_CAUSAL | RA_MOD_SEGMENT | RA_MOD_PREFIX | RA_MOD_WINDOW)) != 0;
  for (int q0 = 0; q0 < p.lq; q0 += BM) {
    load_mod_rows(mt, p.mod, bb, hh, p.lq, q0, ty);
    // A fully masked tile has p = 0 everywhere (finite L): nothing to add.
    if (can_skip && !__syncthreads_or(!patch_all_masked(mt, p.mod, q0, k0, p.lq, p.lk, ty, tx))) continue;
    float s[4][4], dp[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.f;
    for (int dc = 0; dc < p.dk_dim; dc += DC) {   // S = Q K^T
      stage_chunk(As, qb, p.q.sl, q0, p.lq, dc, p.dk_dim, tid);
      stage_chunk(Bs, kb, p.k.sl, k0, p.lk, dc, p.dk_dim, tid);
      __syncthreads();
      mma_chunk(s, As, Bs, ty, tx);
      __syncthreads();
    }
    for (int dc = 0; dc < p.dv_dim; dc += DC) {   // dP = dO V^T
      stage_chunk(As, dob, p.dout.sl, q0, p.lq, dc, p.dv_dim, tid);
      stage_chunk(Bs, vb, p.v.sl, k0, p.lk, dc, p.dv_dim, tid);
      __syncthreads();
      mma_chunk(dp, As, Bs, ty, tx);
      __syncthreads();
    }
    score_tile(s, mt, p.mod, p.scale, bb, hh, q0, k0, p.lq, p.lk, ty, tx);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int row = q0 + ty * 4 + i;
      bool ok = row < p.lq;
      float L = ok ? p.lse[qrow_base + row] : 0.f;
      float dl = ok ? p.delta[qrow_base + row] : 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int col = k0 + tx + 16 * j;
        float pe = 0.f, ds = 0.f;
        if (ok && col < p.lk) {
          // ring.py:146.  With a dense bias tile a row that saw no key (L = -inf) gives
          // exp(-inf + inf) = NaN exactly like the reference; the compiled-in masks
          // define p = 0 on a masked pair, so such rows contribute nothing.
          const bool masked = (s[i][j] == -INFINITY) && !(p.mod.kinds & RA_MOD_DENSE);
          pe = masked ? 0.f : expf(s[i][j] - L);
          ds = masked ? 0.f : pe * (dp[i][j] - dl) * p.scale;  // ring.py:152 (delta is NaN on such rows)
        }
        Ps[(ty * 4 + i) * LDP + tx + 16 * j] = pe;
        Ds[(ty * 4 + i) * LDP + tx + 16 * j] = ds;
      }
    }
    __syncthreads();

    // dV += P^T dO and dK += dS^T Q, 64 columns at a time (ring.py:148, 155).
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const T* src = which == 0 ? dob : qb;
        const int64_t sl = which == 0 ? p.dout.sl : p.q.sl;
        const int dim = which == 0 ? p.dv_dim : p.dk_dim;
        const float* W = which == 0 ? Ps : Ds;
        for (int e = tid; e < 64 * 64; e += NT) {
          int r = e >> 6, c = e & 63;
          float x = 0.f;
          if (q0 + r < p.lq && ch * 64 + c < dim)
            x = load_as_float(src + (int64_t)(q0 + r) * sl + ch * 64 + c);
          Ts[e] = x;
        }
        __syncthreads();
#pragma unroll 4
        for (int qq = 0; qq < BM; ++qq) {
          float w[4], t[JPC];
#pragma unroll
          for (int i = 0; i < 4; ++i) w[i] = W[qq * LDP + ty * 4 + i];
#pragma unroll
          for (int jj = 0; jj < JPC; ++jj) t[jj] = Ts[qq * 64 + tx + 16 * jj];
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int jj = 0; jj < JPC; ++jj) {
              if (which == 0)
                dv_acc[i][ch * JPC + jj] = fmaf(w[i], t[jj], dv_acc[i][ch * JPC + jj]);
              else
                dk_acc[i][ch * JPC + jj] = fmaf(w[i], t[jj], dk_acc[i][ch * JPC + jj]);
            }
        }
        __syncthreads();
      }
      // dQ[:, chunk] = dS K[:, chunk]  (ring.py:154), added to the shared accumulator.
      for (int e = tid; e < 64 * 64; e += NT) {
        int r = e >> 6, c = e & 63;
        float x = 0.f;
        if (k0 + r < p.lk && ch * 64 + c < p.dk_dim)
          x = load_as_float(kb + (int64_t)(k0 + r) * p.k.sl + ch * 64 + c);
        Ts[e] = x;
      }
      __syncthreads();
      float dq_t[4][JPC];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int jj = 0; jj < JPC; ++jj) dq_t[i][jj] = 0.f;
#pragma unroll 4
      for (int kk = 0; kk < BN; ++kk) {
        float w[4], t[JPC];
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = Ds[(ty * 4 + i) * LDP + kk];
#pragma unroll
        for (int jj = 0; jj < JPC; ++jj) t[jj] = Ts[kk * 64 + tx + 16 * jj];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int jj = 0; jj < JPC; ++jj) dq_t[i][jj] = fmaf(w[i], t[jj], dq_t[i][jj]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int row = q0 + ty * 4 + i;
        if (row >= p.lq) continue;
#pragma unroll
        for (int jj = 0; jj < JPC; ++jj) {
          int c = ch * 64 + tx + 16 * jj;
          if (c < p.dk_dim) atomicAdd(p.dq + (qrow_base + row) * p.dk_dim + c, dq_t[i][jj]);
        }
      }
      __syncthreads();
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int row = k0 + ty * 4 + i;
    if (row >= p.lk) continue;
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) {
      int c = tx + 16 * jj;
      if (c < p.dk_dim) p.dk[(krow_base + row) * p.dk_dim + c] += dk_acc[i][jj];
      if (c < p.dv_dim) p.dv[(krow_base + row) * p.dv_dim + c] += dv_acc[i][jj];
    }
  }
}

// ---------------------------------------------------------------------------------------
// Small elementwise kernels.
// ---------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void store_from_float(T* p, float x);
template <>
__device__ __forceinline__ void store_from_float<float>(float* p, float x) {
  *p = x;
}
template <>
__device__ __forceinline__ void store_from_float<__nv_bfloat16>(__nv_bfloat16* p, float x) {
  *p = __float2bfloat16_rn(x);
}

// out = o / l ; L = m + log l (ring.py:134-135).  One warp per row.  With a second state
// (o2, m2, l2) the two are merged first: m = max(m, m2), each side scaled by exp(m_side - m)
// (0 for a side that saw nothing), exactly the update of ring.py:63-75.
template <typename T>
__global__ void finalize_kernel(int b, int h, int lq, int dv, const float* __restrict__ o,
                                const float* __restrict__ m, const float* __restrict__ l,
                                const float* __restrict__ o2, const float* __restrict__ m2,
                                const float* __restrict__ l2, TensorView out, float* __restrict__ lse) {
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  int64_t nrows = (int64_t)b * h * lq;
  if (row >= nrows) return;
  int r = (int)(row % lq);
  int hh = (int)((row / lq) % h);
  int bb = (int)(row / ((int64_t)lq * h));
  float lv = l[row], mv = m[row], c1 = 1.f, c2 = 0.f;
  if (o2) {
    const float ma = mv, mb = m2[row];
    mv = fmaxf(ma, mb);
    c1 = (ma == -INFINITY) ? 0.f : expf(ma - mv);
    c2 = (mb == -INFINITY) ? 0.f : expf(mb - mv);
    lv = lv * c1 + l2[row] * c2;
  }
  if (lane == 0 && lse) lse[row] = mv + logf(lv);
  T* dst = (T*)out.ptr + (int64_t)bb * out.sb + (int64_t)r * out.sl + (int64_t)hh * out.sh;
  for (int c = lane; c < dv; c += 32) {
    float v = o[row * dv + c] * c1;
    if (o2) v += o2[row * dv + c] * c2;
    store_from_float(dst + c, v / lv);
  }
}

// delta = rowsum(out * dout) (ring_kernel.py:387-409; ring.py:151).  One warp per row.
template <typename T>
__global__ void delta_kernel(int b, int h, int lq, int dv, TensorView out, TensorView dout,
                             float* __restrict__ delta) {
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  int64_t nrows = (int64_t)b * h * lq;
  if (row >= nrows) return;
  int r = (int)(row % lq);
  int hh = (int)((row / lq) % h);
  int bb = (int)(row / ((int64_t)lq * h));
  const T* a = (const T*)out.ptr + (int64_t)bb * out.sb + (int64_t)r * out.sl + (int64_t)hh * out.sh;
  const T* g = (const T*)dout.ptr + (int64_t)bb * dout.sb + (int64_t)r * dout.sl + (int64_t)hh * dout.sh;
  float acc = 0.f;
  for (int c = lane; c < dv; c += 32) acc = fmaf(load_as_float(a + c), load_as_float(g + c), acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) delta[row] = acc;
}

template <typename T>
__global__ void cast_kernel(int b, int h, int len, int d, const float* __restrict__ src,
                            TensorView dst) {
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  int64_t nrows = (int64_t)b * h * len;
  if (row >= nrows) return;
  int r = (int)(row % len);
  int hh = (int)((row / len) % h);
  int bb = (int)(row / ((int64_t)len * h));
  T* out = (T*)dst.ptr + (int64_t)bb * dst.sb + (int64_t)r * dst.sl + (int64_t)hh * dst.sh;
  for (int c = lane; c < d; c += 32) store_from_float(out + c, src[row * d + c]);
}

__global__ void add_f32_kernel(float* __restrict__ dst, const float* __restrict__ src, int64_t n) {
  int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
  for (; i + 3 < n; i += stride) {
    float4 a = *reinterpret_cast<float4*>(dst + i);
    float4 c = *reinterpret_cast<const float4*>(src + i);
    a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
    *reinterpret_cast<float4*>(dst + i) = a;
  }
  // tail (n not a multiple of 4): handled by the first threads
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    int64_t j = (n & ~(int64_t)3) + threadIdx.x;
    dst[j] += src[j];
  }
}

__global__ void strict_nan_kernel(int lq, int lk, int dk_dim, int dv_dim, const float* __restrict__ lse,
                                  float* __restrict__ dq, float* __restrict__ dk, float* __restrict__ dv) {
  const int64_t bh = blockIdx.x;
  const float* L = lse + bh * lq;
  const float nan = __int_as_float(0x7fc00000);
  int any = 0;
  for (int i = threadIdx.x; i < lq; i += blockDim.x)
    if (L[i] == -INFINITY) any = 1;
  any = __syncthreads_or(any);
  if (!any) return;
  float* dq_bh = dq + bh * lq * dk_dim;
  for (int64_t e = threadIdx.x; e < (int64_t)lq * dk_dim; e += blockDim.x)
    if (L[e / dk_dim] == -INFINITY) dq_bh[e] = nan;
  float* dk_bh = dk + bh * lk * dk_dim;
  for (int64_t e = threadIdx.x; e < (int64_t)lk * dk_dim; e += blockDim.x) dk_bh[e] = nan;
  float* dv_bh = dv + bh * lk * dv_dim;
  for (int64_t e = threadIdx.x; e < (int64_t)lk * dv_dim; e += blockDim.x) dv_bh[e] = nan;
}

template <typename T, int D_PAD>
cudaError_t launch_fwd(const FwdParams& p, cudaStream_t s) {
  size_t smem = sizeof(float) * (2 * 64 * LDS + 64 * LDP + 64 * D_PAD);
  auto kern = simt_fwd_kernel<T, D_PAD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid((p.lq + BM - 1) / BM, p.h, p.b);
  kern<<<grid, NT, smem, s>>>(p);
  count_launch();
  return cudaGetLastError();
}

template <typename T, int D_PAD>
cudaError_t launch_bwd(const BwdParams& p, cudaStream_t s) {
  size_t smem = sizeof(float) * (2 * 64 * LDS + 2 * 64 * LDP + 64 * 64);
  auto kern = simt_bwd_kernel<T, D_PAD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid((p.lk + BN - 1) / BN, p.h, p.b);
  kern<<<grid, NT, smem, s>>>(p);
  count_launch();
  return cudaGetLastError();
}

template <typename T>
cudaError_t dispatch_fwd(const FwdParams& p, cudaStream_t s) {
  int d = p.dv;
  if (d <= 16) return launch_fwd<T, 16>(p, s);
  if (d <= 64) return launch_fwd<T, 64>(p, s);
  if (d <= 128) return launch_fwd<T, 128>(p, s);
  return launch_fwd<T, 256>(p, s);
}
template <typename T>
cudaError_t dispatch_bwd(const BwdParams& p, cudaStream_t s) {
  int d = p.dk_dim > p.dv_dim ? p.dk_dim : p.dv_dim;
  if (d <= 16) return launch_bwd<T, 16>(p, s);
  if (d <= 64) return launch_bwd<T, 64>(p, s);
  if (d <= 128) return launch_bwd<T, 128>(p, s);
  return launch_bwd<T, 256>(p, s);
}

}  // namespace

cudaError_t simt_fwd_block(const FwdParams& p, int dtype, cudaStream_t s) {
  return dtype == RA_DTYPE_F32 ? dispatch_fwd<float>(p, s) : dispatch_fwd<__nv_bfloat16>(p, s);
}
cudaError_t simt_bwd_block(const BwdParams& p, int dtype, cudaStream_t s) {
  return dtype == RA_DTYPE_F32 ? dispatch_bwd<float>(p, s) : dispatch_bwd<__nv_bfloat16>(p, s);
}

cudaError_t launch_finalize(int b, int h, int lq, int dv, const float* o, const float* m, const float* l,
                            const float* o2, const float* m2, const float* l2, TensorView out, int dtype,
                            float* lse, cudaStream_t s) {
  int64_t rows = (int64_t)b * h * lq;
  int grid = (int)((rows + 7) / 8);
  if (dtype == RA_DTYPE_F32)
    finalize_kernel<float><<<grid, 256, 0, s>>>(b, h, lq, dv, o, m, l, o2, m2, l2, out, lse);
  else
    finalize_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(b, h, lq, dv, o, m, l, o2, m2, l2, out, lse);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_delta(int b, int h, int lq, int dv, TensorView out, TensorView dout, int dtype,
                         float* delta, cudaStream_t s) {
  int64_t rows = (int64_t)b * h * lq;
  int grid = (int)((rows + 7) / 8);
  if (dtype == RA_DTYPE_F32)
    delta_kernel<float><<<grid, 256, 0, s>>>(b, h, lq, dv, out, dout, delta);
  else
    delta_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(b, h, lq, dv, out, dout, delta);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_cast_from_f32(int b, int h, int len, int d, const float* src, TensorView dst,
                                 int dtype, cudaStream_t s) {
  int64_t rows = (int64_t)b * h * len;
  int grid = (int)((rows + 7) / 8);
  if (dtype == RA_DTYPE_F32)
    cast_kernel<float><<<grid, 256, 0, s>>>(b, h, len, d, src, dst);
  else
    cast_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(b, h, len, d, src, dst);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_strict_nan(int b, int h, int lq, int lk, int dk_dim, int dv_dim, const float* lse, float* dq,
                              float* dk, float* dv, cudaStream_t s) {
  strict_nan_kernel<<<b * h, 512, 0, s>>>(lq, lk, dk_dim, dv_dim, lse, dq, dk, dv);
  count_launch();
  return cudaGetLastError();
}

__global__ void bwd_row_terms_kernel(const float* __restrict__ lse, const float* __restrict__ delta, float scale,
                                     int clamp, int64_t n, float* __restrict__ nl2, float* __restrict__ nds) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float x = -lse[i] * 1.4426950408889634f;
  nl2[i] = clamp ? fminf(x, 1e30f) : x;
  nds[i] = -delta[i] * scale;
}

__global__ void add_rows_f32_kernel(float* __restrict__ dst, const float* __restrict__ src, int64_t seg_elems,
                                    int64_t pitch) {
  float* d = dst + (int64_t)blockIdx.y * pitch;
  const float* c = src + (int64_t)blockIdx.y * pitch;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i + 3 < seg_elems; i += (int64_t)gridDim.x * blockDim.x * 4) {
    float4 a = *reinterpret_cast<float4*>(d + i);
    const float4 x = *reinterpret_cast<const float4*>(c + i);
    a.x += x.x, a.y += x.y, a.z += x.z, a.w += x.w;
    *reinterpret_cast<float4*>(d + i) = a;
  }
}

cudaError_t launch_bwd_row_terms(const float* lse, const float* delta, float scale, int clamp, int64_t n, float* nl2,
                                 float* nds, cudaStream_t s) {
  bwd_row_terms_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(lse, delta, scale, clamp, n, nl2, nds);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_add_rows_f32(float* dst, const float* src, int64_t nseg, int64_t seg_elems, int64_t pitch, cudaStream_t s) {
  if (nseg <= 0 || seg_elems <= 0) return cudaSuccess;
  if (seg_elems % 4 || pitch % 4 || nseg > 65535) {  // odd sizes: one flat add per segment
    for (int64_t g = 0; g < nseg; ++g) {
      cudaError_t e = launch_add_f32(dst + g * pitch, src + g * pitch, seg_elems, s);
      if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
  }
  int64_t want = (seg_elems / 4 + 255) / 256;
  dim3 grid((unsigned)(want > 64 ? 64 : want), (unsigned)nseg);
  add_rows_f32_kernel<<<grid, 256, 0, s>>>(dst, src, seg_elems, pitch);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_add_f32(float* dst, const float* src, int64_t n, cudaStream_t s) {
  int64_t want = (n / 4 + 255) / 256;
  int grid = (int)(want < 1 ? 1 : (want > 148 * 8 ? 148 * 8 : want));
  add_f32_kernel<<<grid, 256, 0, s>>>(dst, src, n);
  count_launch();
  return cudaGetLastError();
}

}  // namespace ra
