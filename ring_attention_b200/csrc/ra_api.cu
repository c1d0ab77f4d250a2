// C ABI of the engine: argument checks, kernel-family dispatch, error strings.
// The ring schedule lives in ring.cu; the kernels in simt_kernels.cu and *_sm100.cu.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "host_util.h"
#include "tc_common.cuh"

namespace ra {

static thread_local char g_err[512] = "";
static thread_local int g_impl = RA_IMPL_AUTO;
static thread_local int g_last_impl = 0;
static std::atomic<int64_t> g_launches{0};

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
int fail_cuda(cudaError_t e, const char* what) {
  return fail(RA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}
int current_impl() { return g_impl; }
void set_last_impl(int impl) { g_last_impl = impl; }
int last_impl() { return g_last_impl; }

static TensorView view(const ra_tensor_t* t) {
  return TensorView{t->ptr, t->stride_b, t->stride_l, t->stride_h};
}

int check_shape(const ra_shape_t* s) {
  if (!s) return fail(-1, "shape is NULL");
  if (s->b < 1 || s->h < 1 || s->lq < 1 || s->lk < 1 || s->dk < 1 || s->dv < 1)
    return fail(-2, "shape: b,h,lq,lk,dk,dv must all be >= 1 (got %d,%d,%d,%d,%d,%d)", s->b, s->h,
                s->lq, s->lk, s->dk, s->dv);
  if (s->dk > 256 || s->dv > 256) return fail(-3, "head dims above 256 are not supported");
  if (s->dtype != RA_DTYPE_F32 && s->dtype != RA_DTYPE_BF16)
    return fail(-4, "dtype must be RA_DTYPE_F32 or RA_DTYPE_BF16 (got %d)", s->dtype);
  if (!(s->sm_scale == s->sm_scale)) return fail(-5, "sm_scale is NaN");
  return 0;
}
int check_tensor(const ra_tensor_t* t, const char* name) {
  if (!t || !t->ptr) return fail(-6, "tensor %s is NULL", name);
  return 0;
}
int check_mod(const ra_score_mod_t* m, ModParams* out) {
  memset(out, 0, sizeof(*out));
  if (!m) return 0;
  const uint32_t known = RA_MOD_CAUSAL | RA_MOD_SEGMENT | RA_MOD_PREFIX | RA_MOD_ALIBI |
                         RA_MOD_WINDOW | RA_MOD_DENSE | RA_MOD_STRICT_NAN;
  if (m->kinds & ~known) return fail(-7, "score_mod: unknown kind bits 0x%x", m->kinds & ~known);
  // The same combinations ring_self_attention refuses (ring.py:368-374).
  if ((m->kinds & RA_MOD_CAUSAL) && (m->kinds & RA_MOD_PREFIX))
    return fail(-8, "score_mod: causal attention does not support prefix_mask");
  const uint32_t needs_pos = RA_MOD_CAUSAL | RA_MOD_PREFIX | RA_MOD_ALIBI | RA_MOD_WINDOW;
  if ((m->kinds & needs_pos) && (!m->q_pos || !m->kv_pos))
    return fail(-9, "score_mod: positions are required for causal/prefix/alibi/window");
  if ((m->kinds & RA_MOD_SEGMENT) && (!m->q_seg || !m->kv_seg))
    return fail(-10, "score_mod: segment ids are required for RA_MOD_SEGMENT");
  if ((m->kinds & RA_MOD_PREFIX) && (!m->q_prefix || !m->kv_prefix))
    return fail(-11, "score_mod: prefix masks are required for RA_MOD_PREFIX");
  if ((m->kinds & RA_MOD_ALIBI) && !m->alibi_slopes)
    return fail(-12, "score_mod: alibi_slopes is NULL");
  if ((m->kinds & RA_MOD_WINDOW) && m->window < 1) return fail(-13, "score_mod: window must be >= 1");
  if ((m->kinds & RA_MOD_DENSE) && !m->bias) return fail(-14, "score_mod: dense bias is NULL");
  out->kinds = m->kinds;
  out->window = m->window;
  out->q_pos = m->q_pos;
  out->kv_pos = m->kv_pos;
  out->q_seg = m->q_seg;
  out->kv_seg = m->kv_seg;
  out->q_pre = m->q_prefix;
  out->kv_pre = m->kv_prefix;
  out->slopes = m->alibi_slopes;
  out->bias = m->bias;
  out->bsb = m->bias_stride_b;
  out->bsh = m->bias_stride_h;
  out->bsq = m->bias_stride_q;
  return 0;
}

// Runs one forward block with whichever family applies.  Shared with ring.cu.
int run_fwd_block(const FwdParams& p, int dtype, cudaStream_t s) {
  int impl = g_impl;
  if (impl != RA_IMPL_SIMT) {
    const char* why = tc_fwd_unsupported_reason(p, dtype);
    if (!why) {
      cudaError_t e = tc_fwd_block(p, s);
      if (e == cudaSuccess) {
        g_last_impl = RA_IMPL_TCGEN05;
        return 0;
      }
      // cudaErrorNotSupported: the driver refused a tensor map for these strides
      if (e != cudaErrorNotSupported || impl == RA_IMPL_TCGEN05) return fail_cuda(e, "tcgen05 forward block");
    }
    if (why && impl == RA_IMPL_TCGEN05) return fail(-20, "tcgen05 forward does not take this call: %s", why);
  }
  cudaError_t e = simt_fwd_block(p, dtype, s);
  if (e != cudaSuccess) return fail_cuda(e, "simt forward block");
  g_last_impl = RA_IMPL_SIMT;
  return 0;
}

// ring.py:146 on a row whose L is -inf: see RA_MOD_STRICT_NAN.  Runs after the block kernel, on
// the fp32 accumulators the block added into.
static int strict_nan(const BwdParams& p, cudaStream_t s) {
  if (!(p.mod.kinds & RA_MOD_STRICT_NAN) || (p.mod.kinds & RA_MOD_DENSE)) return 0;
  cudaError_t e = launch_strict_nan(p.b, p.h, p.lq, p.lk, p.dk_dim, p.dv_dim, p.lse, p.dq, p.dk, p.dv, s);
  if (e != cudaSuccess) return fail_cuda(e, "strict NaN pass");
  return 0;
}

int run_bwd_block(const BwdParams& p, int dtype, cudaStream_t s) {
  int impl = g_impl;
  if ((p.mod.kinds & RA_MOD_STRICT_NAN) && p.dk_out.ptr)
    return fail(-44, "RA_MOD_STRICT_NAN needs the fp32 accumulators, not direct results");
  if (impl != RA_IMPL_SIMT) {
    const char* why = tc_bwd_unsupported_reason(p, dtype);
    if (!why) {
      cudaError_t e = tc_bwd_block(p, s);
      if (e == cudaSuccess) {
        g_last_impl = RA_IMPL_TCGEN05;
        return strict_nan(p, s);
      }
      if (e != cudaErrorNotSupported || impl == RA_IMPL_TCGEN05) return fail_cuda(e, "tcgen05 backward block");
    }
    if (why && impl == RA_IMPL_TCGEN05) return fail(-20, "tcgen05 backward does not take this call: %s", why);
  }
  if (p.overwrite) {  // the CUDA-core kernel adds: clear what the caller left uncleared
    cudaError_t e = cudaMemsetAsync(p.dk, 0, (size_t)p.b * p.h * p.lk * p.dk_dim * sizeof(float), s);
    if (e == cudaSuccess) e = cudaMemsetAsync(p.dv, 0, (size_t)p.b * p.h * p.lk * p.dv_dim * sizeof(float), s);
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync");
    count_launch(2);
  }
  cudaError_t e = simt_bwd_block(p, dtype, s);
  if (e != cudaSuccess) return fail_cuda(e, "simt backward block");
  g_last_impl = RA_IMPL_SIMT;
  return strict_nan(p, s);
}

}  // namespace ra

using namespace ra;

extern "C" {

int ra_version(void) { return RA_VERSION; }
const char* ra_last_error_string(void) { return g_err; }
int ra_set_impl(int impl) {
  if (impl < RA_IMPL_AUTO || impl > RA_IMPL_TCGEN05) return fail(-21, "unknown impl %d", impl);
  g_impl = impl;
  return 0;
}
int ra_last_impl(void) { return g_last_impl; }
int64_t ra_launch_count(void) { return g_launches.load(); }

int ra_device_status(uint32_t* bits) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceSynchronize");
  unsigned int* word = device_status_word();
  if (!word) return fail(RA_ERR_CUDA, "status word symbol not found");
  unsigned int v = 0, zero = 0;
  if ((e = cudaMemcpy(&v, word, sizeof(v), cudaMemcpyDeviceToHost)) != cudaSuccess) return fail_cuda(e, "cudaMemcpy");
  if (v && (e = cudaMemcpy(word, &zero, sizeof(zero), cudaMemcpyHostToDevice)) != cudaSuccess)
    return fail_cuda(e, "cudaMemcpy");
  if (bits) *bits = v;
  if (v) return fail(RA_ERR_DEVICE_STATUS, "a bounded wait ran out inside a kernel (status bits 0x%x)", v);
  return 0;
}

int ra_fwd_block(const ra_shape_t* shape, const ra_tensor_t* q, const ra_tensor_t* k,
                 const ra_tensor_t* v, const ra_score_mod_t* mod, float* o, float* m, float* l,
                 int first, void* stream) {
  int rc;
  if ((rc = check_shape(shape))) return rc;
  if ((rc = check_tensor(q, "q")) || (rc = check_tensor(k, "k")) || (rc = check_tensor(v, "v")))
    return rc;
  if (!o || !m || !l) return fail(-6, "carried state (o, m, l) is NULL");
  FwdParams p;
  memset(&p, 0, sizeof(p));
  if ((rc = check_mod(mod, &p.mod))) return rc;
  p.q = view(q);
  p.k = view(k);
  p.v = view(v);
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
  return run_fwd_block(p, shape->dtype, (cudaStream_t)stream);
}

int ra_fwd_finalize(const ra_shape_t* shape, const float* o, const float* m, const float* l,
                    const ra_tensor_t* out, float* lse, void* stream) {
  int rc;
  if ((rc = check_shape(shape))) return rc;
  if ((rc = check_tensor(out, "out"))) return rc;
  if (!o || !m || !l) return fail(-6, "carried state (o, m, l) is NULL");
  cudaError_t e = launch_finalize(shape->b, shape->h, shape->lq, shape->dv, o, m, l, nullptr, nullptr, nullptr, view(out),
                                  shape->dtype, lse, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail_cuda(e, "finalize");
  return 0;
}

int ra_bwd_delta(const ra_shape_t* shape, const ra_tensor_t* out, const ra_tensor_t* dout,
                 float* delta, void* stream) {
  int rc;
  if ((rc = check_shape(shape))) return rc;
  if ((rc = check_tensor(out, "out")) || (rc = check_tensor(dout, "dout"))) return rc;
  if (!delta) return fail(-6, "delta is NULL");
  cudaError_t e = launch_delta(shape->b, shape->h, shape->lq, shape->dv, view(out), view(dout),
                               shape->dtype, delta, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail_cuda(e, "delta");
  return 0;
}

int ra_bwd_block(const ra_shape_t* shape, const ra_tensor_t* q, const ra_tensor_t* k,
                 const ra_tensor_t* v, const ra_score_mod_t* mod, const float* lse,
                 const float* delta, const ra_tensor_t* dout, float* dq, float* dk, float* dv,
                 void* stream) {
  int rc;
  if ((rc = check_shape(shape))) return rc;
  if ((rc = check_tensor(q, "q")) || (rc = check_tensor(k, "k")) || (rc = check_tensor(v, "v")) ||
      (rc = check_tensor(dout, "dout")))
    return rc;
  if (!lse || !delta || !dq || !dk || !dv) return fail(-6, "lse/delta/dq/dk/dv is NULL");
  BwdParams p;
  memset(&p, 0, sizeof(p));
  if ((rc = check_mod(mod, &p.mod))) return rc;
  p.q = view(q);
  p.k = view(k);
  p.v = view(v);
  p.dout = view(dout);
  p.lse = lse;
  p.delta = delta;
  p.dq = dq;
  p.dk = dk;
  p.dv = dv;
  p.b = shape->b;
  p.h = shape->h;
  p.lq = shape->lq;
  p.lk = shape->lk;
  p.dk_dim = shape->dk;
  p.dv_dim = shape->dv;
  p.scale = shape->sm_scale;
  return run_bwd_block(p, shape->dtype, (cudaStream_t)stream);
}

int ra_cast_from_f32(int32_t b, int32_t h, int32_t len, int32_t d, const float* src,
                     const ra_tensor_t* dst, int32_t dtype, void* stream) {
  int rc;
  if (b < 1 || h < 1 || len < 1 || d < 1) return fail(-2, "cast: sizes must be >= 1");
  if (!src) return fail(-6, "cast: src is NULL");
  if ((rc = check_tensor(dst, "dst"))) return rc;
  if (dtype != RA_DTYPE_F32 && dtype != RA_DTYPE_BF16) return fail(-4, "cast: bad dtype %d", dtype);
  cudaError_t e = launch_cast_from_f32(b, h, len, d, src, view(dst), dtype, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail_cuda(e, "cast");
  return 0;
}

}  // extern "C"
