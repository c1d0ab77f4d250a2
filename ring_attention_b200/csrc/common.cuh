// Internal parameter blocks shared by the host dispatcher and the kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ring_attention_b200.h"
#include "score_mod.h"

namespace ra {

struct TensorView {
  const void* ptr;
  int64_t sb, sl, sh;  // element strides of batch, length, heads; head_dim stride is 1
};

struct ModParams {
  uint32_t kinds;
  int32_t window;
  const int32_t* q_pos;
  const int32_t* kv_pos;
  const int32_t* q_seg;
  const int32_t* kv_seg;
  const uint8_t* q_pre;
  const uint8_t* kv_pre;
  const float* slopes;
  const float* bias;
  int64_t bsb, bsh, bsq;
};

struct FwdParams {
  TensorView q, k, v;
  ModParams mod;
  float* o;  // [b,h,lq,dv] fp32, un-normalised
  float* m;  // [b,h,lq]
  float* l;  // [b,h,lq]
  int32_t b, h, lq, lk, dk, dv;
  float scale;
  int32_t first;
  // Optional, honoured by the tcgen05 kernel only: when final_out.ptr is set this is the last
  // block of the attention, and the kernel writes out = o / l (input dtype) and L = m + log l
  // (ring.py:134-135) itself instead of storing the carried state.
  TensorView final_out;
  float* final_lse;
};

struct BwdParams {
  TensorView q, k, v, dout;
  ModParams mod;
  const float* lse;    // [b,h,lq]
  const float* delta;  // [b,h,lq]
  // Optional, read by the tcgen05 kernel instead of lse / delta when set: the per-row terms of
  // its inner loops, computed once per backward instead of once per tile and thread:
  //   row_nl2 = min(-lse * log2(e), 1e30)  (no clamp with a dense bias tile: ring.py:146 as it is)
  //   row_nds = -delta * scale
  // When they are NULL the launcher derives them into scratch first.
  const float* row_nl2;
  const float* row_nds;
  float* dq;           // [b,h,lq,dk] fp32, accumulated with atomics
  float* dk;           // [b,h,lk,dk] fp32, += per call
  float* dv;           // [b,h,lk,dv] fp32, += per call
  int32_t b, h, lq, lk, dk_dim, dv_dim;
  float scale;
  // Optional, honoured by the tcgen05 kernel only: when dk_out.ptr is set this call is the
  // whole backward for these keys (ring of one) and the kernel stores dK, dV in the input
  // dtype straight to the result tensors; dk / dv above are then not touched.
  TensorView dk_out, dv_out;
  // Optional: dk / dv above hold nothing yet and this call defines them (stores instead of
  // read-add-write, zeros for key rows that no query sees), so the caller need not clear them.
  // The tcgen05 kernel does it in its epilogue; for the CUDA-core kernel the dispatcher clears first.
  int32_t overwrite;
};

// Launchers implemented in the .cu files.  Each returns a cudaError_t.
cudaError_t simt_fwd_block(const FwdParams& p, int dtype, cudaStream_t s);
cudaError_t simt_bwd_block(const BwdParams& p, int dtype, cudaStream_t s);
// out = o / l, L = m + log l (ring.py:134-135).  With o2 != NULL the two carried states are
// merged first, as one more online-softmax update (ring.py:63-75) would.
cudaError_t launch_finalize(int b, int h, int lq, int dv, const float* o, const float* m, const float* l,
                            const float* o2, const float* m2, const float* l2, TensorView out, int dtype,
                            float* lse, cudaStream_t s);
cudaError_t launch_delta(int b, int h, int lq, int dv, TensorView out, TensorView dout, int dtype,
                         float* delta, cudaStream_t s);
cudaError_t launch_cast_from_f32(int b, int h, int len, int d, const float* src, TensorView dst,
                                 int dtype, cudaStream_t s);
// nl2[i] = min(-lse[i] * log2(e), 1e30) (clamp left out when !clamp), nds[i] = -delta[i] * scale.
cudaError_t launch_bwd_row_terms(const float* lse, const float* delta, float scale, int clamp, int64_t n, float* nl2,
                                 float* nds, cudaStream_t s);
cudaError_t launch_add_f32(float* dst, const float* src, int64_t n, cudaStream_t s);
// dst[seg * pitch + i] += src[seg * pitch + i] for seg < nseg, i < seg_elems (a multiple of 4; 16-byte aligned rows).
cudaError_t launch_add_rows_f32(float* dst, const float* src, int64_t nseg, int64_t seg_elems, int64_t pitch, cudaStream_t s);
// One block per (batch, head): where some query row has L = -inf, dq of those rows and all of
// dk, dv of that (batch, head) become NaN (what ring.py:146 produces for such rows).
cudaError_t launch_strict_nan(int b, int h, int lq, int lk, int dk_dim, int dv_dim, const float* lse, float* dq,
                              float* dk, float* dv, cudaStream_t s);

void count_launch(int n = 1);

// Score-mod inputs of one token (a query row or a key row).
struct ModRow {
  int32_t pos, seg;
  bool pre;
};

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) {
  return *p;
}
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}

}  // namespace ra
