// Ring schedule: one process per GPU.  The forward follows ring_attention/ring.py:79-137
// and the backward ring.py:160-211, with two changes that NVSwitch makes free:
//   * at step t a rank works on the K/V block of rank (rank - t) mod N, exactly the
//     block the reference's hop-by-hop ppermute (ring.py:54) would have delivered, but
//     the owner sends it straight to its consumer (no forwarding hop), into the half of
//     a double buffer that the running block kernel is not reading;
//   * in the backward K/V are fetched the same way, dQ stays at home, and the dK/dV
//     contribution of a step goes straight to the block's owner, which adds it in fp32.
// Transfers are NCCL send/recv on a side stream, fenced against the caller's stream
// with events; nothing here synchronises the host.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "host_util.h"

namespace ra {

namespace {

// NCCL is resolved at run time so that the library loads on machines without it
// (single-GPU use needs no NCCL at all).
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi* nccl_api() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api.handle ? &api : nullptr;
  tried = true;
  const char* env = getenv("RA_NCCL_LIB");
  const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    if (!n) continue;
    api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (api.handle) break;
  }
  if (!api.handle) return nullptr;
#define RA_SYM(field, name)                                                \
  api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, name)); \
  if (!api.field) {                                                        \
    api.handle = nullptr;                                                  \
    return nullptr;                                                        \
  }
  RA_SYM(GetUniqueId, "ncclGetUniqueId")
  RA_SYM(CommInitRank, "ncclCommInitRank")
  RA_SYM(CommDestroy, "ncclCommDestroy")
  RA_SYM(Send, "ncclSend")
  RA_SYM(Recv, "ncclRecv")
  RA_SYM(GroupStart, "ncclGroupStart")
  RA_SYM(GroupEnd, "ncclGroupEnd")
  RA_SYM(GetErrorString, "ncclGetErrorString")
#undef RA_SYM
  return &api;
}

int fail_nccl(ncclResult_t r, const char* what) {
  NcclApi* api = nccl_api();
  return fail(RA_ERR_NCCL, "%s: %s", what, api ? api->GetErrorString(r) : "NCCL not loaded");
}

struct Buffer {
  void* ptr = nullptr;
  size_t bytes = 0;
  // Grow-only device buffer.  Growing synchronises the device, so steady-state calls
  // with a fixed shape never allocate.
  cudaError_t reserve(size_t n) {
    if (n <= bytes) return cudaSuccess;
    if (ptr) {
      cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) return e;
      cudaFree(ptr);
      ptr = nullptr;
      bytes = 0;
    }
    cudaError_t e = cudaMalloc(&ptr, n);
    if (e == cudaSuccess) bytes = n;
    return e;
  }
  void release() {
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    bytes = 0;
  }
};

size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

// A tensor is "dense" when its b*len*h*d elements occupy exactly that many consecutive
// elements (in any order of b, len, h): only then can it be sent as one flat message and
// read on the other side with the same strides.
bool is_dense(const TensorView& t, int b, int len, int h, int d) {
  int64_t dims[3] = {b, len, h};
  int64_t str[3] = {t.sb, t.sl, t.sh};
  for (int i = 0; i < 3; ++i)
    for (int j = i + 1; j < 3; ++j)
      if (str[j] < str[i]) {
        std::swap(str[i], str[j]);
        std::swap(dims[i], dims[j]);
      }
  int64_t expect = d;
  for (int i = 0; i < 3; ++i) {
    if (dims[i] == 1) continue;
    if (str[i] != expect) return false;
    expect *= dims[i];
  }
  return true;
}

}  // namespace

}  // namespace ra

using namespace ra;

struct ra_ring {
  int rank = 0, nranks = 1, device = 0;
  ncclComm_t comm = nullptr;
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ev_start = nullptr, ev_recv[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr};
  cudaEvent_t ev_part[2] = {nullptr, nullptr}, ev_sent[2] = {nullptr, nullptr}, ev_tail = nullptr;
  Buffer state;    // o (fp32), m, l
  Buffer stage[2]; // K, V and the kv-side score-mod arrays of a remote block
  Buffer grads;    // delta, dq, dk, dv accumulators (fp32)
  Buffer part[2];  // this rank's dK/dV contribution for a remote block
  Buffer rpart[2]; // a remote rank's contribution for this rank's block
  bool timing = false;
  // timing, kept per direction ([0] forward call, [1] backward call)
  std::vector<cudaEvent_t> t_events[2];  // pairs bracketing each wait on a transfer
  std::vector<cudaEvent_t> b_events[2];  // pairs bracketing each block-kernel launch
  cudaEvent_t t_begin[2] = {nullptr, nullptr}, t_end[2] = {nullptr, nullptr};
  size_t t_used[2] = {0, 0}, b_used[2] = {0, 0};
  int dir = 0;  // direction of the call in progress
};

namespace {

struct KvMessage {
  // Flat messages that make up one K/V block: pointers on the sender (own tensors) and
  // byte sizes; the receiver lays them out back to back in a staging buffer.
  const void* src[5];
  size_t bytes[5];
  size_t offset[5];
  int n = 0;
  size_t total = 0;
  void add(const void* p, size_t nbytes) {
    src[n] = p;
    bytes[n] = nbytes;
    offset[n] = total;
    total += align_up(nbytes);
    ++n;
  }
};

KvMessage make_kv_message(const ra_shape_t* sh, const TensorView& k, const TensorView& v,
                          const ModParams& mod) {
  KvMessage msg;
  size_t es = sh->dtype == RA_DTYPE_F32 ? 4 : 2;
  msg.add(k.ptr, (size_t)sh->b * sh->lk * sh->h * sh->dk * es);
  msg.add(v.ptr, (size_t)sh->b * sh->lk * sh->h * sh->dv * es);
  size_t tok = (size_t)sh->b * sh->lk;
  if (mod.kv_pos) msg.add(mod.kv_pos, tok * 4);
  if (mod.kv_seg) msg.add(mod.kv_seg, tok * 4);
  if (mod.kv_pre) msg.add(mod.kv_pre, tok);
  return msg;
}

// Point the kv side of (k, v, mod) at a staged block.
void use_staged(const KvMessage& msg, void* base, TensorView* k, TensorView* v, ModParams* mod) {
  char* p = (char*)base;
  int i = 0;
  k->ptr = p + msg.offset[i++];
  v->ptr = p + msg.offset[i++];
  if (mod->kv_pos) mod->kv_pos = (const int32_t*)(p + msg.offset[i++]);
  if (mod->kv_seg) mod->kv_seg = (const int32_t*)(p + msg.offset[i++]);
  if (mod->kv_pre) mod->kv_pre = (const uint8_t*)(p + msg.offset[i++]);
}

int exchange_kv(ra_ring_t* r, const KvMessage& msg, void* stage, int to, int from) {
  NcclApi* api = nccl_api();
  ncclResult_t rc = api->GroupStart();
  if (rc != ncclSuccess) return fail_nccl(rc, "ncclGroupStart");
  for (int i = 0; i < msg.n; ++i) {
    rc = api->Send(msg.src[i], msg.bytes[i], ncclChar, to, r->comm, r->comm_stream);
    if (rc != ncclSuccess) return fail_nccl(rc, "ncclSend");
    rc = api->Recv((char*)stage + msg.offset[i], msg.bytes[i], ncclChar, from, r->comm, r->comm_stream);
    if (rc != ncclSuccess) return fail_nccl(rc, "ncclRecv");
  }
  rc = api->GroupEnd();
  if (rc != ncclSuccess) return fail_nccl(rc, "ncclGroupEnd");
  return 0;
}

#define RA_CUDA(call, what)                             \
  do {                                                  \
    cudaError_t e__ = (call);                           \
    if (e__ != cudaSuccess) return fail_cuda(e__, what); \
  } while (0)

int timing_mark(ra_ring_t* r, cudaStream_t s) {
  if (!r->timing) return 0;
  const int d = r->dir;
  if (r->t_used[d] == r->t_events[d].size()) {
    cudaEvent_t e;
    RA_CUDA(cudaEventCreate(&e), "cudaEventCreate");
    r->t_events[d].push_back(e);
  }
  RA_CUDA(cudaEventRecord(r->t_events[d][r->t_used[d]++], s), "cudaEventRecord");
  return 0;
}

int block_mark(ra_ring_t* r, int dir, cudaStream_t s) {
  if (!r->timing) return 0;
  if (r->b_used[dir] == r->b_events[dir].size()) {
    cudaEvent_t e;
    RA_CUDA(cudaEventCreate(&e), "cudaEventCreate");
    r->b_events[dir].push_back(e);
  }
  RA_CUDA(cudaEventRecord(r->b_events[dir][r->b_used[dir]++], s), "cudaEventRecord");
  return 0;
}

// Make the caller's stream wait for a transfer; with timing on, bracket the wait.
int wait_transfer(ra_ring_t* r, cudaStream_t s, cudaEvent_t ev) {
  int rc;
  if ((rc = timing_mark(r, s))) return rc;
  RA_CUDA(cudaStreamWaitEvent(s, ev, 0), "cudaStreamWaitEvent");
  if ((rc = timing_mark(r, s))) return rc;
  return 0;
}

int check_ring_call(ra_ring_t* ring, const ra_shape_t* shape, const TensorView& k,
                    const TensorView& v) {
  if (!ring) return fail(-30, "ring handle is NULL");
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (dev != ring->device)
    return fail(-31, "ring was created on device %d but device %d is current", ring->device, dev);
  if (ring->nranks > 1) {
    if (!is_dense(k, shape->b, shape->lk, shape->h, shape->dk) ||
        !is_dense(v, shape->b, shape->lk, shape->h, shape->dv))
      return fail(-32, "with more than one rank k and v must be dense (no gaps between elements)");
  }
  return 0;
}

}  // namespace

extern "C" {

int ra_ring_source(int32_t rank, int32_t nranks, int32_t step) {
  if (nranks < 1 || rank < 0 || rank >= nranks || step < 0) return fail(-33, "bad rank/nranks/step");
  return ((rank - step) % nranks + nranks) % nranks;
}

int ra_ring_unique_id(uint8_t id[RA_UNIQUE_ID_BYTES]) {
  static_assert(sizeof(ncclUniqueId) == RA_UNIQUE_ID_BYTES, "unique id size");
  NcclApi* api = nccl_api();
  if (!api) return fail(RA_ERR_NCCL, "NCCL library not found (set RA_NCCL_LIB to libnccl.so.2)");
  ncclUniqueId uid;
  ncclResult_t rc = api->GetUniqueId(&uid);
  if (rc != ncclSuccess) return fail_nccl(rc, "ncclGetUniqueId");
  memcpy(id, &uid, sizeof(uid));
  return 0;
}

int ra_ring_create(int32_t rank, int32_t nranks, const uint8_t nccl_id[RA_UNIQUE_ID_BYTES],
                   ra_ring_t** out) {
  if (!out) return fail(-30, "ring out-pointer is NULL");
  if (nranks < 1 || rank < 0 || rank >= nranks) return fail(-33, "bad rank %d of %d", rank, nranks);
  ra_ring_t* r = new ra_ring_t();
  r->rank = rank;
  r->nranks = nranks;
  cudaError_t e = cudaGetDevice(&r->device);
  if (e != cudaSuccess) {
    delete r;
    return fail_cuda(e, "cudaGetDevice");
  }
  auto bail = [&](int code) {
    ra_ring_destroy(r);
    return code;
  };
  if ((e = cudaStreamCreateWithFlags(&r->comm_stream, cudaStreamNonBlocking)) != cudaSuccess)
    return bail(fail_cuda(e, "cudaStreamCreate"));
  cudaEvent_t* evs[] = {&r->ev_start, &r->ev_recv[0], &r->ev_recv[1], &r->ev_done[0], &r->ev_done[1],
                        &r->ev_part[0], &r->ev_part[1], &r->ev_sent[0], &r->ev_sent[1], &r->ev_tail};
  for (cudaEvent_t* ev : evs)
    if ((e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming)) != cudaSuccess)
      return bail(fail_cuda(e, "cudaEventCreate"));
  for (int d = 0; d < 2; ++d)
    if ((e = cudaEventCreate(&r->t_begin[d])) != cudaSuccess || (e = cudaEventCreate(&r->t_end[d])) != cudaSuccess)
      return bail(fail_cuda(e, "cudaEventCreate"));
  if (nranks > 1) {
    if (!nccl_id) return bail(fail(-34, "nccl_id is NULL with nranks > 1"));
    NcclApi* api = nccl_api();
    if (!api) return bail(fail(RA_ERR_NCCL, "NCCL library not found (set RA_NCCL_LIB to libnccl.so.2)"));
    ncclUniqueId uid;
    memcpy(&uid, nccl_id, sizeof(uid));
    ncclResult_t rc = api->CommInitRank(&r->comm, nranks, uid, rank);
    if (rc != ncclSuccess) return bail(fail_nccl(rc, "ncclCommInitRank"));
  }
  *out = r;
  return 0;
}

int ra_ring_destroy(ra_ring_t* r) {
  if (!r) return 0;
  if (r->comm_stream) cudaStreamSynchronize(r->comm_stream);
  if (r->comm) {
    NcclApi* api = nccl_api();
    if (api) api->CommDestroy(r->comm);
  }
  cudaEvent_t evs[] = {r->ev_start, r->ev_recv[0], r->ev_recv[1], r->ev_done[0], r->ev_done[1],
                       r->ev_part[0], r->ev_part[1], r->ev_sent[0], r->ev_sent[1], r->ev_tail,
                       r->t_begin[0], r->t_begin[1], r->t_end[0], r->t_end[1]};
  for (cudaEvent_t ev : evs)
    if (ev) cudaEventDestroy(ev);
  for (int d = 0; d < 2; ++d) {
    for (cudaEvent_t ev : r->t_events[d]) cudaEventDestroy(ev);
    for (cudaEvent_t ev : r->b_events[d]) cudaEventDestroy(ev);
  }
  if (r->comm_stream) cudaStreamDestroy(r->comm_stream);
  r->state.release();
  r->grads.release();
  for (int i = 0; i < 2; ++i) {
    r->stage[i].release();
    r->part[i].release();
    r->rpart[i].release();
  }
  delete r;
  return 0;
}

int ra_ring_rank(const ra_ring_t* r) { return r ? r->rank : fail(-30, "ring handle is NULL"); }
int ra_ring_size(const ra_ring_t* r) { return r ? r->nranks : fail(-30, "ring handle is NULL"); }

int ra_ring_set_timing(ra_ring_t* r, int32_t on) {
  if (!r) return fail(-30, "ring handle is NULL");
  r->timing = on != 0;
  return 0;
}

int ra_ring_last_timing(ra_ring_t* r, int32_t backward, float* total_ms, float* exposed_ms) {
  if (!r) return fail(-30, "ring handle is NULL");
  if (!r->timing) return fail(-35, "timing is off: call ra_ring_set_timing(ring, 1) first");
  const int d = backward ? 1 : 0;
  RA_CUDA(cudaEventSynchronize(r->t_end[d]), "cudaEventSynchronize");
  float tot = 0.f, exp = 0.f;
  RA_CUDA(cudaEventElapsedTime(&tot, r->t_begin[d], r->t_end[d]), "cudaEventElapsedTime");
  for (size_t i = 0; i + 1 < r->t_used[d]; i += 2) {
    float ms = 0.f;
    RA_CUDA(cudaEventElapsedTime(&ms, r->t_events[d][i], r->t_events[d][i + 1]), "cudaEventElapsedTime");
    exp += ms;
  }
  if (total_ms) *total_ms = tot;
  if (exposed_ms) *exposed_ms = exp;
  return 0;
}

int ra_ring_last_block_ms(ra_ring_t* r, int32_t backward, float* block_ms, int32_t* launches) {
  if (!r) return fail(-30, "ring handle is NULL");
  if (!r->timing) return fail(-35, "timing is off: call ra_ring_set_timing(ring, 1) first");
  const int dir = backward ? 1 : 0;
  if (r->b_used[dir] == 0) return fail(-38, "no %s call has been timed yet", dir ? "backward" : "forward");
  RA_CUDA(cudaEventSynchronize(r->t_end[dir]), "cudaEventSynchronize");
  float sum = 0.f;
  for (size_t i = 0; i + 1 < r->b_used[dir]; i += 2) {
    float ms = 0.f;
    RA_CUDA(cudaEventElapsedTime(&ms, r->b_events[dir][i], r->b_events[dir][i + 1]), "cudaEventElapsedTime");
    sum += ms;
  }
  if (block_ms) *block_ms = sum;
  if (launches) *launches = (int32_t)(r->b_used[dir] / 2);
  return 0;
}

int ra_ring_fwd(ra_ring_t* ring, const ra_shape_t* shape, const ra_tensor_t* q,
                const ra_tensor_t* k, const ra_tensor_t* v, const ra_score_mod_t* mod,
                const ra_tensor_t* out, float* lse, void* stream_) {
  int rc;
  cudaStream_t stream = (cudaStream_t)stream_;
  if ((rc = check_shape(shape))) return rc;
  if ((rc = check_tensor(q, "q")) || (rc = check_tensor(k, "k")) || (rc = check_tensor(v, "v")) ||
      (rc = check_tensor(out, "out")))
    return rc;
  FwdParams p;
  memset(&p, 0, sizeof(p));
  if ((rc = check_mod(mod, &p.mod))) return rc;
  if (p.mod.kinds & RA_MOD_DENSE)
    return fail(-36, "a dense bias tile cannot travel round the ring; use the block-level calls");
  p.q = {q->ptr, q->stride_b, q->stride_l, q->stride_h};
  p.k = {k->ptr, k->stride_b, k->stride_l, k->stride_h};
  p.v = {v->ptr, v->stride_b, v->stride_l, v->stride_h};
  if ((rc = check_ring_call(ring, shape, p.k, p.v))) return rc;
  const int N = ring->nranks, me = ring->rank;
  p.b = shape->b;
  p.h = shape->h;
  p.lq = shape->lq;
  p.lk = shape->lk;
  p.dk = shape->dk;
  p.dv = shape->dv;
  p.scale = shape->sm_scale;

  const size_t rows = (size_t)shape->b * shape->h * shape->lq;
  const size_t o_bytes = align_up(rows * shape->dv * 4), ml_bytes = align_up(rows * 4);
  RA_CUDA(ring->state.reserve(o_bytes + 2 * ml_bytes), "cudaMalloc(state)");
  p.o = (float*)ring->state.ptr;
  p.m = (float*)((char*)ring->state.ptr + o_bytes);
  p.l = (float*)((char*)ring->state.ptr + o_bytes + ml_bytes);

  KvMessage msg = make_kv_message(shape, p.k, p.v, p.mod);
  if (N > 1) {
    RA_CUDA(ring->stage[0].reserve(msg.total), "cudaMalloc(stage)");
    RA_CUDA(ring->stage[1].reserve(msg.total), "cudaMalloc(stage)");
    // transfers read the caller's K/V: order them after whatever produced those
    RA_CUDA(cudaEventRecord(ring->ev_start, stream), "cudaEventRecord");
    RA_CUDA(cudaStreamWaitEvent(ring->comm_stream, ring->ev_start, 0), "cudaStreamWaitEvent");
  }
  ring->dir = 0;
  ring->t_used[0] = 0;
  ring->b_used[0] = 0;
  if (ring->timing) RA_CUDA(cudaEventRecord(ring->t_begin[0], stream), "cudaEventRecord");

  const TensorView k_own = p.k, v_own = p.v;
  const ModParams mod_own = p.mod;
  for (int t = 0; t < N; ++t) {
    if (t + 1 < N) {  // fetch the block of step t+1 while step t computes
      int slot = (t + 1) & 1;
      if (t >= 1) RA_CUDA(cudaStreamWaitEvent(ring->comm_stream, ring->ev_done[slot], 0), "cudaStreamWaitEvent");
      int to = (me + t + 1) % N, from = ((me - t - 1) % N + N) % N;
      if ((rc = exchange_kv(ring, msg, ring->stage[slot].ptr, to, from))) return rc;
      RA_CUDA(cudaEventRecord(ring->ev_recv[slot], ring->comm_stream), "cudaEventRecord");
    }
    p.k = k_own;
    p.v = v_own;
    p.mod = mod_own;
    if (t > 0) {
      use_staged(msg, ring->stage[t & 1].ptr, &p.k, &p.v, &p.mod);
      if ((rc = wait_transfer(ring, stream, ring->ev_recv[t & 1]))) return rc;
    }
    p.first = (t == 0);
    if ((rc = block_mark(ring, 0, stream))) return rc;
    if ((rc = run_fwd_block(p, shape->dtype, stream))) return rc;
    if ((rc = block_mark(ring, 0, stream))) return rc;
    if (N > 1) RA_CUDA(cudaEventRecord(ring->ev_done[t & 1], stream), "cudaEventRecord");
  }
  cudaError_t e = launch_finalize(shape->b, shape->h, shape->lq, shape->dv, p.o, p.m, p.l,
                                  TensorView{out->ptr, out->stride_b, out->stride_l, out->stride_h},
                                  shape->dtype, lse, stream);
  if (e != cudaSuccess) return fail_cuda(e, "finalize");
  if (ring->timing) RA_CUDA(cudaEventRecord(ring->t_end[0], stream), "cudaEventRecord");
  return 0;
}

int ra_ring_bwd(ra_ring_t* ring, const ra_shape_t* shape, const ra_tensor_t* q,
                const ra_tensor_t* k, const ra_tensor_t* v, const ra_tensor_t* out,
                const float* lse, const ra_tensor_t* dout, const ra_score_mod_t* mod,
                const ra_tensor_t* dq, const ra_tensor_t* dk, const ra_tensor_t* dv,
                void* stream_) {
  int rc;
  cudaStream_t stream = (cudaStream_t)stream_;
  if ((rc = check_shape(shape))) return rc;
  if ((rc = check_tensor(q, "q")) || (rc = check_tensor(k, "k")) || (rc = check_tensor(v, "v")) ||
      (rc = check_tensor(out, "out")) || (rc = check_tensor(dout, "dout")) ||
      (rc = check_tensor(dq, "dq")) || (rc = check_tensor(dk, "dk")) || (rc = check_tensor(dv, "dv")))
    return rc;
  if (!lse) return fail(-6, "lse is NULL");
  BwdParams p;
  memset(&p, 0, sizeof(p));
  if ((rc = check_mod(mod, &p.mod))) return rc;
  if (p.mod.kinds & RA_MOD_DENSE)
    return fail(-36, "a dense bias tile cannot travel round the ring; use the block-level calls");
  auto tv = [](const ra_tensor_t* t) { return TensorView{t->ptr, t->stride_b, t->stride_l, t->stride_h}; };
  p.q = tv(q);
  p.k = tv(k);
  p.v = tv(v);
  p.dout = tv(dout);
  if ((rc = check_ring_call(ring, shape, p.k, p.v))) return rc;
  const int N = ring->nranks, me = ring->rank;
  p.b = shape->b;
  p.h = shape->h;
  p.lq = shape->lq;
  p.lk = shape->lk;
  p.dk_dim = shape->dk;
  p.dv_dim = shape->dv;
  p.scale = shape->sm_scale;
  p.lse = lse;

  const size_t qrows = (size_t)shape->b * shape->h * shape->lq;
  const size_t krows = (size_t)shape->b * shape->h * shape->lk;
  const size_t delta_b = align_up(qrows * 4), dq_b = align_up(qrows * shape->dk * 4);
  const size_t dk_b = align_up(krows * shape->dk * 4), dv_b = align_up(krows * shape->dv * 4);
  RA_CUDA(ring->grads.reserve(delta_b + dq_b + dk_b + dv_b), "cudaMalloc(grads)");
  char* g = (char*)ring->grads.ptr;
  float* delta = (float*)g;
  float* dq_acc = (float*)(g + delta_b);
  float* dk_acc = (float*)(g + delta_b + dq_b);
  float* dv_acc = (float*)(g + delta_b + dq_b + dk_b);
  KvMessage msg = make_kv_message(shape, p.k, p.v, p.mod);
  if (N > 1) {
    for (int i = 0; i < 2; ++i) {
      RA_CUDA(ring->stage[i].reserve(msg.total), "cudaMalloc(stage)");
      RA_CUDA(ring->part[i].reserve(dk_b + dv_b), "cudaMalloc(part)");
      RA_CUDA(ring->rpart[i].reserve(dk_b + dv_b), "cudaMalloc(rpart)");
    }
    RA_CUDA(cudaEventRecord(ring->ev_start, stream), "cudaEventRecord");
    RA_CUDA(cudaStreamWaitEvent(ring->comm_stream, ring->ev_start, 0), "cudaStreamWaitEvent");
  }
  ring->dir = 1;
  ring->t_used[1] = 0;
  ring->b_used[1] = 0;
  if (ring->timing) RA_CUDA(cudaEventRecord(ring->t_begin[1], stream), "cudaEventRecord");

  cudaError_t e = launch_delta(shape->b, shape->h, shape->lq, shape->dv, tv(out), p.dout,
                               shape->dtype, delta, stream);
  if (e != cudaSuccess) return fail_cuda(e, "delta");
  p.delta = delta;
  p.dq = dq_acc;
  RA_CUDA(cudaMemsetAsync(dq_acc, 0, dq_b + dk_b + dv_b, stream), "cudaMemsetAsync");
  count_launch();

  NcclApi* api = N > 1 ? nccl_api() : nullptr;
  const TensorView k_own = p.k, v_own = p.v;
  const ModParams mod_own = p.mod;
  for (int t = 0; t < N; ++t) {
    if (t + 1 < N) {
      int slot = (t + 1) & 1;
      if (t >= 1) RA_CUDA(cudaStreamWaitEvent(ring->comm_stream, ring->ev_done[slot], 0), "cudaStreamWaitEvent");
      int to = (me + t + 1) % N, from = ((me - t - 1) % N + N) % N;
      if ((rc = exchange_kv(ring, msg, ring->stage[slot].ptr, to, from))) return rc;
      RA_CUDA(cudaEventRecord(ring->ev_recv[slot], ring->comm_stream), "cudaEventRecord");
    }
    p.k = k_own;
    p.v = v_own;
    p.mod = mod_own;
    if (t == 0) {
      p.dk = dk_acc;
      p.dv = dv_acc;
      if ((rc = block_mark(ring, 1, stream))) return rc;
      if ((rc = run_bwd_block(p, shape->dtype, stream))) return rc;
      if ((rc = block_mark(ring, 1, stream))) return rc;
      if (N > 1) RA_CUDA(cudaEventRecord(ring->ev_done[0], stream), "cudaEventRecord");
      continue;
    }
    const int slot = t & 1;
    use_staged(msg, ring->stage[slot].ptr, &p.k, &p.v, &p.mod);
    if ((rc = wait_transfer(ring, stream, ring->ev_recv[slot]))) return rc;
    // this step's contribution to the remote block's dK/dV, built from zero
    if (t >= 3) RA_CUDA(cudaStreamWaitEvent(stream, ring->ev_sent[slot], 0), "cudaStreamWaitEvent");
    p.dk = (float*)ring->part[slot].ptr;
    p.dv = (float*)((char*)ring->part[slot].ptr + dk_b);
    RA_CUDA(cudaMemsetAsync(ring->part[slot].ptr, 0, dk_b + dv_b, stream), "cudaMemsetAsync");
    count_launch();
    if ((rc = block_mark(ring, 1, stream))) return rc;
    if ((rc = run_bwd_block(p, shape->dtype, stream))) return rc;
    if ((rc = block_mark(ring, 1, stream))) return rc;
    RA_CUDA(cudaEventRecord(ring->ev_done[slot], stream), "cudaEventRecord");
    RA_CUDA(cudaEventRecord(ring->ev_part[slot], stream), "cudaEventRecord");
    // send it to the block's owner; receive what another rank computed for our block
    RA_CUDA(cudaStreamWaitEvent(ring->comm_stream, ring->ev_part[slot], 0), "cudaStreamWaitEvent");
    int owner = ((me - t) % N + N) % N, giver = (me + t) % N;
    ncclResult_t nr = api->GroupStart();
    if (nr != ncclSuccess) return fail_nccl(nr, "ncclGroupStart");
    nr = api->Send(ring->part[slot].ptr, dk_b + dv_b, ncclChar, owner, ring->comm, ring->comm_stream);
    if (nr != ncclSuccess) return fail_nccl(nr, "ncclSend");
    nr = api->Recv(ring->rpart[slot].ptr, dk_b + dv_b, ncclChar, giver, ring->comm, ring->comm_stream);
    if (nr != ncclSuccess) return fail_nccl(nr, "ncclRecv");
    nr = api->GroupEnd();
    if (nr != ncclSuccess) return fail_nccl(nr, "ncclGroupEnd");
    RA_CUDA(cudaEventRecord(ring->ev_sent[slot], ring->comm_stream), "cudaEventRecord");
    e = launch_add_f32(dk_acc, (const float*)ring->rpart[slot].ptr, (int64_t)((dk_b + dv_b) / 4),
                       ring->comm_stream);
    if (e != cudaSuccess) return fail_cuda(e, "add");
  }
  if (N > 1) {
    RA_CUDA(cudaEventRecord(ring->ev_tail, ring->comm_stream), "cudaEventRecord");
    if ((rc = wait_transfer(ring, stream, ring->ev_tail))) return rc;
  }
  if ((e = launch_cast_from_f32(shape->b, shape->h, shape->lq, shape->dk, dq_acc, tv(dq), shape->dtype, stream)) != cudaSuccess ||
      (e = launch_cast_from_f32(shape->b, shape->h, shape->lk, shape->dk, dk_acc, tv(dk), shape->dtype, stream)) != cudaSuccess ||
      (e = launch_cast_from_f32(shape->b, shape->h, shape->lk, shape->dv, dv_acc, tv(dv), shape->dtype, stream)) != cudaSuccess)
    return fail_cuda(e, "cast");
  if (ring->timing) RA_CUDA(cudaEventRecord(ring->t_end[1], stream), "cudaEventRecord");
  return 0;
}

int ra_ring_rotate(ra_ring_t* ring, int32_t n, const void* const* src, void* const* dst,
                   const int64_t* nbytes, void* stream_) {
  if (!ring) return fail(-30, "ring handle is NULL");
  if (n < 0 || (n > 0 && (!src || !dst || !nbytes))) return fail(-37, "rotate: bad buffer lists");
  cudaStream_t stream = (cudaStream_t)stream_;
  if (ring->nranks == 1) {
    for (int i = 0; i < n; ++i)
      if (src[i] != dst[i])
        RA_CUDA(cudaMemcpyAsync(dst[i], src[i], (size_t)nbytes[i], cudaMemcpyDeviceToDevice, stream), "cudaMemcpyAsync");
    return 0;
  }
  NcclApi* api = nccl_api();
  const int N = ring->nranks, to = (ring->rank + 1) % N, from = (ring->rank + N - 1) % N;
  ncclResult_t nr = api->GroupStart();
  if (nr != ncclSuccess) return fail_nccl(nr, "ncclGroupStart");
  for (int i = 0; i < n; ++i) {
    if (nbytes[i] <= 0) continue;
    nr = api->Send(src[i], (size_t)nbytes[i], ncclChar, to, ring->comm, stream);
    if (nr != ncclSuccess) return fail_nccl(nr, "ncclSend");
    nr = api->Recv(dst[i], (size_t)nbytes[i], ncclChar, from, ring->comm, stream);
    if (nr != ncclSuccess) return fail_nccl(nr, "ncclRecv");
  }
  nr = api->GroupEnd();
  if (nr != ncclSuccess) return fail_nccl(nr, "ncclGroupEnd");
  return 0;
}

}  // extern "C"
