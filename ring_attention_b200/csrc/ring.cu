// Ring schedule: one process per GPU.  The forward follows ring_attention/ring.py:79-137
// and the backward ring.py:160-211, with these changes that NVSwitch makes free:
//   * at step t a rank works on the K/V block of rank (rank - t) mod N, exactly the
//     block the reference's hop-by-hop ppermute (ring.py:54) would have delivered, but
//     the owner sends it straight to its consumer (no forwarding hop), into one of four
//     staging slots (slot = step mod 4);
//   * in the backward K/V are fetched the same way, dQ stays at home, and the dK/dV
//     contribution of a step goes straight to the block's owner, which adds it in fp32;
//   * the block kernels of adjacent steps run on two compute lanes (the caller's stream and a
//     second stream), so that the tail of one overlaps the head of the next: the forward keeps
//     one carried state per lane and merges them at the end, the backward's steps share only
//     the dQ accumulator, which is added to with reductions.
// Two transports:
//   p2p  (default): the owner PUSHES with copy-engine peer copies (cudaMemcpyAsync into the
//         consumer's staging slot, mapped through CUDA IPC) on high-priority side streams (one
//         for K/V blocks, one for contributions): no SM is used, so the copy really runs under
//         the block kernel.  Ordering between GPUs uses 64-bit sequence counters in each rank's
//         flag page, written with release stores by small kernels after the copy and polled with
//         acquire loads by small bounded-wait kernels on the stream that needs the data.
//   nccl: grouped ncclSend / ncclRecv on the side stream (RA_TRANSPORT=nccl, or chosen by every
//         rank together when some rank cannot map a peer).  Its fixed cost per exchange (~0.4 ms
//         measured at 8 GPUs) is too high for short ring steps.
// Nothing here synchronises the host, except when buffers have to grow (ra_ring_reserve does
// that ahead of time).
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <utility>
#include <vector>

#include "common.cuh"
#include "host_util.h"
#include "tc_common.cuh"

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
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
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
  RA_SYM(AllGather, "ncclAllGather")
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

namespace ringimpl {

// Flag page of one rank (64-bit counters, all monotonic over the life of the ring).
//   KV_READY[slot]   written by the rank that pushed a K/V block into stage[slot]: global step id
//   PART_READY[slot] written by the rank that pushed a dK/dV contribution into rpart[slot]
//   PROGRESS[lane][j] written by rank j: global id up to which j has finished the block steps of
//                    one compute lane (frees that lane's stage slot)
//   ADDED[j]         written by rank j: global id up to which j has summed received contributions
// Block steps alternate between two compute lanes (even steps on the caller's stream, odd steps
// on a second compute stream of the ring), so that the tail of one block kernel overlaps the
// head of the next; a step's staging slot, contribution buffer, forward state and PROGRESS
// counter are those of its lane (slot = lane = step parity), and steps of one lane stay ordered.
constexpr int kMaxRanks = 64;
// Staging slots for incoming K/V blocks, buffers for outgoing and for incoming dK/dV
// contributions: slot = step % kSlots.  Two would do for one compute lane; with two lanes the
// blocks of steps t and t+1 are both in use while the block of step t+2 should already be
// travelling, and a contribution buffer must not wait for its predecessor's transfer.
constexpr int kSlots = 4;
constexpr int kFlagKvReady = 0, kFlagPartReady = 4, kFlagProgress = 8, kFlagAdded = 8 + 2 * kMaxRanks;
constexpr int kNumFlags = 8 + 3 * kMaxRanks;
constexpr int progress_flag(int lane, int rank) { return kFlagProgress + lane * kMaxRanks + rank; }
constexpr uint32_t kStRingWait = 1u << 16;  // status bit: a cross-GPU wait ran out

struct FlagList {
  uint64_t* ptr[kMaxRanks];
  int n;
};

// One thread; waits until *flag >= target.  Bounded: gives up after max_cycles SM cycles,
// records it in the status word, raises the ring's abort word and returns, so the stream
// always drains.  Once the abort word is up every later wait of the ring returns at once.
__global__ void wait_flag_kernel(const uint64_t* flag, uint64_t target, unsigned int* status, unsigned int* abort_word,
                                 long long max_cycles) {
  if (*(volatile unsigned int*)abort_word) return;
  const long long t0 = clock64();
  while (true) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
    if (v >= target) return;
    __nanosleep(100);
    if (clock64() - t0 > max_cycles) {
      atomicOr(status, kStRingWait);
      atomicExch(abort_word, 1u);
      __threadfence();
      return;
    }
  }
}

// Thread i publishes `value` to list.ptr[i] (own or peer memory) after everything that
// preceded this kernel on its stream -- unless a wait of this ring has run out: what the
// stream did after that wait may have used a block that never arrived or overwritten one
// that was still being read, and must not be announced as ready.  The peers' own waits then
// run out in turn, so the failure is reported on every rank instead of spreading as data.
__global__ void set_flags_kernel(FlagList list, uint64_t value, const unsigned int* abort_word) {
  const int i = threadIdx.x;
  if (i >= list.n) return;
  if (*(volatile const unsigned int*)abort_word) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(list.ptr[i]), "l"(value) : "memory");
}

struct IpcBundle {
  cudaIpcMemHandle_t stage[kSlots], rpart[kSlots], flags;
};

}  // namespace ringimpl
using namespace ringimpl;

// Which (query shard, K/V block) pairs of the ring have a visible pair at all: need[q_rank * n + kv_rank].
// rows: for every pair, up to two runs of K/V rows (one in each half of the block: a zig-zag
// shard is two position-contiguous halves) outside which the queries of q_rank see nothing,
// in 128-row chunks: rows[((q_rank * n + kv_rank) * 2 + half) * 2 + {0: first, 1: one past last}].
struct ra_ring_plan {
  int nranks = 1;
  int lk = 0;  // K/V rows per block the row runs were computed for (0: no runs, whole blocks move)
  std::vector<uint8_t> need;
  std::vector<int32_t> rows;
};

struct ra_ring {
  int rank = 0, nranks = 1, device = 0;
  const ra_ring_plan* plan = nullptr;  // not owned; NULL: every step runs
  bool ignore_plan = false;            // the call in progress runs every step (RA_MOD_STRICT_NAN)
  ncclComm_t comm = nullptr;
  cudaStream_t push_stream = nullptr;    // transfers this rank issues (high priority)
  cudaStream_t reduce_stream = nullptr;  // sums of dK/dV contributions this rank receives (p2p)
  cudaStream_t lane_stream = nullptr;    // second compute lane: the odd block steps
  // dK/dV contributions this rank gives (p2p): a stream of their own, so that the K/V block of a
  // later step never queues behind a contribution that waits for its block kernel.  With the
  // NCCL transport it is the transfer stream itself (one communicator, one stream).
  cudaStream_t give_stream = nullptr;
  cudaEvent_t ev_give_tail = nullptr;
  // PROGRESS counters are published from this high-priority stream, behind an event of the lane:
  // a one-thread kernel on a lane itself queues behind the other lane's block kernel until that
  // kernel's last wave, and the peers' pushes would start that much later.
  cudaStream_t flag_stream = nullptr;
  cudaEvent_t ev_main_end = nullptr;
  cudaEvent_t ev_lane_start = nullptr, ev_lane_done = nullptr;
  cudaEvent_t ev_start = nullptr, ev_recv[ringimpl::kSlots] = {}, ev_done[ringimpl::kSlots] = {};
  cudaEvent_t ev_part[ringimpl::kSlots] = {}, ev_sent[ringimpl::kSlots] = {}, ev_tail = nullptr;
  cudaEvent_t ev_push_tail = nullptr, ev_step0 = nullptr;
  bool p2p = false;
  // buffers other ranks write into (cudaMalloc'ed, exported through CUDA IPC under p2p)
  void* stage[ringimpl::kSlots] = {};  // K, V and the kv-side score-mod arrays of a remote block
  void* rpart[ringimpl::kSlots] = {};  // a remote rank's dK/dV contribution for this rank's block
  size_t stage_bytes = 0, rpart_bytes = 0;
  uint64_t* flags = nullptr;
  // [0] abort word: set by a wait that ran out, checked by every later wait and flag store of
  // this ring; [2..3] a 64-bit counter nothing ever advances (ra_ring_probe_wait)
  unsigned int* guard = nullptr;
  long long wait_cycles = 0;  // bound of one wait for a peer, in SM cycles
  struct Peer {
    void* stage[ringimpl::kSlots] = {};
    void* rpart[ringimpl::kSlots] = {};
    uint64_t* flags = nullptr;
  };
  std::vector<Peer> peers;  // this process's view of every rank's buffers ([rank] = own pointers)
  void* ipc_send = nullptr;  // device scratch for the handle all-gather
  void* ipc_recv = nullptr;
  uint64_t epoch = 0;  // global step id of the next call's step 0 (advances by nranks per call)
  Buffer state;    // o (fp32), m, l
  Buffer grads;    // delta, dq, dk, dv accumulators (fp32)
  Buffer part[ringimpl::kSlots];  // this rank's dK/dV contributions for remote blocks
  bool timing = false;
  // timing, kept per direction ([0] forward call, [1] backward call)
  std::vector<cudaEvent_t> t_events[2];  // pairs bracketing each wait on a transfer
  std::vector<cudaEvent_t> b_events[2];  // pairs bracketing each block-kernel launch
  cudaEvent_t t_begin[2] = {nullptr, nullptr}, t_end[2] = {nullptr, nullptr};
  size_t t_used[2] = {0, 0}, b_used[2] = {0, 0};
  std::vector<cudaEvent_t> p_events[2];  // pairs bracketing each transfer this rank issues
  size_t p_used[2] = {0, 0};
  double p_bytes[2] = {0, 0};            // bytes this rank sent in the last call of each direction
  int dir = 0;  // direction of the call in progress
};

namespace ringimpl {

// Position / segment / prefix summary of each run of 128 tokens (the last one may be shorter):
// one warp per chunk.  Same fields as the block kernels' tile summaries, any length.
__global__ void plan_meta_kernel(TileMeta* __restrict__ out, const int32_t* __restrict__ pos,
                                 const int32_t* __restrict__ seg, const uint8_t* __restrict__ pre, int len, int n_chunks) {
  const int chunk = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31, bb = blockIdx.y;
  if (chunk >= n_chunks) return;
  const int64_t base = (int64_t)bb * len;
  int pmin = INT32_MAX, pmax = INT32_MIN, smin = INT32_MAX, smax = INT32_MIN, any = 0, all = 1;
  for (int e = chunk * 128 + lane; e < len && e < chunk * 128 + 128; e += 32) {
    if (pos) {
      const int v = pos[base + e];
      pmin = min(pmin, v);
      pmax = max(pmax, v);
    }
    if (seg) {
      const int v = seg[base + e];
      smin = min(smin, v);
      smax = max(smax, v);
    }
    if (pre) {
      const int v = pre[base + e] != 0;
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
  }
  if (lane == 0) {
    TileMeta m;
    m.pos_min = pos ? pmin : 0;
    m.pos_max = pos ? pmax : 0;
    m.seg_min = seg ? smin : 0;
    m.seg_max = seg ? smax : 0;
    m.pre_any = pre ? any : 0;
    m.pre_all = pre ? all : 0;
    m.pos_contig = 0;
    m.pad1 = 0;
    out[(int64_t)bb * n_chunks + chunk] = m;
  }
}

// all: [nranks][b * (nq + nk)] summaries, the q chunks of a rank first.  For the pair (r, o) =
// (blockIdx.x / nranks, blockIdx.x % nranks): need = 1 when some query chunk of rank r and some
// K/V chunk of rank o (same batch element) are not fully masked, and rows[pair][half] = the run
// [first, one past last] of such K/V chunks in each half of the block (over all batch elements).
__global__ void plan_need_kernel(const TileMeta* __restrict__ all, int nranks, int b, int nq, int nk, uint32_t kinds,
                                 int32_t window, int* __restrict__ need, int32_t* __restrict__ rows) {
  const int r = blockIdx.x / nranks, o = blockIdx.x % nranks;
  const int64_t per_rank = (int64_t)b * (nq + nk);
  const TileMeta* mq = all + r * per_rank;
  const TileMeta* mk = all + o * per_rank + (int64_t)b * nq;
  __shared__ int s_lo[2], s_hi[2];
  if (threadIdx.x < 2) {
    s_lo[threadIdx.x] = INT32_MAX;
    s_hi[threadIdx.x] = 0;
  }
  __syncthreads();
  const int half_at = (nk + 1) / 2;
  for (int i = threadIdx.x; i < b * nk; i += blockDim.x) {
    const int bb = i / nk, kc = i % nk;
    const TileMeta k = mk[bb * nk + kc];
    bool seen = false;
    for (int qc = 0; qc < nq && !seen; ++qc) seen = classify_tiles(kinds, window, mq[bb * nq + qc], k) != 0;
    if (seen) {
      const int half = kc >= half_at ? 1 : 0;
      atomicMin(&s_lo[half], kc);
      atomicMax(&s_hi[half], kc + 1);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    need[blockIdx.x] = (s_hi[0] > 0 || s_hi[1] > 0) ? 1 : 0;
    for (int half = 0; half < 2; ++half) {
      rows[blockIdx.x * 4 + half * 2] = s_hi[half] > 0 ? s_lo[half] : 0;
      rows[blockIdx.x * 4 + half * 2 + 1] = s_hi[half];
    }
  }
}

struct KvMessage {
  // Flat messages that make up one K/V block: pointers on the sender (own tensors) and
  // byte sizes; the receiver lays them out back to back in a staging buffer.
  const void* src[5];
  size_t bytes[5];
  size_t offset[5];
  // parts that are [b][lk rows][row_bytes] and may travel as row runs: bytes of one row (0: the
  // part always travels whole) and number of batch elements
  size_t row_bytes[5];
  int nb[5];
  int n = 0;
  size_t total = 0;
  void add(const void* p, size_t nbytes, size_t row = 0, int batches = 1) {
    src[n] = p;
    bytes[n] = nbytes;
    offset[n] = total;
    row_bytes[n] = row;
    nb[n] = batches;
    total += align_up(nbytes);
    ++n;
  }
};

// Up to two runs of K/V rows of one block.
struct RowRuns {
  int n = 1;
  int lo[2] = {0, 0}, hi[2] = {0, 0};
};

KvMessage make_kv_message(const ra_shape_t* sh, const TensorView& k, const TensorView& v,
                          const ModParams& mod) {
  KvMessage msg;
  size_t es = sh->dtype == RA_DTYPE_F32 ? 4 : 2;
  // row runs need rows that are contiguous and batch elements one block of rows apart: [b, l, h, d]
  auto blhd = [&](const TensorView& t, int d) {
    return (sh->h == 1 || t.sh == d) && (sh->lk == 1 || t.sl == (int64_t)sh->h * d) &&
           (sh->b == 1 || t.sb == (int64_t)sh->lk * sh->h * d);
  };
  msg.add(k.ptr, (size_t)sh->b * sh->lk * sh->h * sh->dk * es, blhd(k, sh->dk) ? (size_t)sh->h * sh->dk * es : 0, sh->b);
  msg.add(v.ptr, (size_t)sh->b * sh->lk * sh->h * sh->dv * es, blhd(v, sh->dv) ? (size_t)sh->h * sh->dv * es : 0, sh->b);
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

#define RA_CUDA(call, what)                             \
  do {                                                  \
    cudaError_t e__ = (call);                           \
    if (e__ != cudaSuccess) return fail_cuda(e__, what); \
  } while (0)
#define RA_NCCL(call, what)                                  \
  do {                                                       \
    ncclResult_t r__ = (call);                               \
    if (r__ != ncclSuccess) return fail_nccl(r__, what);     \
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

// How long a rank waits for a peer before it gives up (the peer may simply be late: another
// stream of work, a slow host), counted in SM cycles at 2 GHz.
long long wait_cycles_of_ms(long long ms) {
  if (ms < 1) ms = 1;
  if (ms > 600000) ms = 600000;
  return ms * 2000000LL;
}

// Brackets one outgoing transfer on the transfer stream (timing on only).
int push_mark(ra_ring_t* r, cudaStream_t s, double bytes) {
  if (!r->timing) return 0;
  const int d = r->dir;
  if (r->p_used[d] == r->p_events[d].size()) {
    cudaEvent_t e;
    RA_CUDA(cudaEventCreate(&e), "cudaEventCreate");
    r->p_events[d].push_back(e);
  }
  RA_CUDA(cudaEventRecord(r->p_events[d][r->p_used[d]++], s), "cudaEventRecord");
  r->p_bytes[d] += bytes;
  return 0;
}

int launch_wait(ra_ring_t* r, cudaStream_t s, int flag_index, uint64_t target) {
  unsigned int* status = device_status_word();
  if (!status) return fail(RA_ERR_CUDA, "status word symbol not found");
  wait_flag_kernel<<<1, 1, 0, s>>>(r->flags + flag_index, target, status, r->guard, r->wait_cycles);
  count_launch();
  RA_CUDA(cudaGetLastError(), "wait_flag_kernel");
  return 0;
}

// Publish `value` into flag `flag_index` of one peer (peer >= 0) or of every rank but this one (-1).
int launch_set(ra_ring_t* r, cudaStream_t s, int peer, int flag_index, uint64_t value) {
  FlagList list;
  list.n = 0;
  for (int j = 0; j < r->nranks; ++j) {
    if (peer >= 0 ? j != peer : j == r->rank) continue;
    list.ptr[list.n++] = r->peers[j].flags + flag_index;
  }
  if (list.n == 0) return 0;
  set_flags_kernel<<<1, kMaxRanks, 0, s>>>(list, value, r->guard);
  count_launch();
  RA_CUDA(cudaGetLastError(), "set_flags_kernel");
  return 0;
}

// Make the caller's stream wait for an event recorded on a transfer stream; with timing on,
// bracket the wait.
int wait_transfer(ra_ring_t* r, cudaStream_t s, cudaEvent_t ev) {
  int rc;
  if ((rc = timing_mark(r, s))) return rc;
  RA_CUDA(cudaStreamWaitEvent(s, ev, 0), "cudaStreamWaitEvent");
  if ((rc = timing_mark(r, s))) return rc;
  return 0;
}

void close_peers(ra_ring_t* r) {
  for (int j = 0; j < (int)r->peers.size(); ++j) {
    if (j == r->rank) continue;
    ra_ring::Peer& p = r->peers[j];
    for (int i = 0; i < kSlots; ++i) {
      if (p.stage[i]) cudaIpcCloseMemHandle(p.stage[i]);
      if (p.rpart[i]) cudaIpcCloseMemHandle(p.rpart[i]);
      p.stage[i] = p.rpart[i] = nullptr;
    }
    if (p.flags) cudaIpcCloseMemHandle(p.flags);
    p.flags = nullptr;
  }
}

// Sizes of everything a ring call keeps in the handle, from the shape alone.
struct RingSizes {
  size_t o_bytes, ml_bytes;                                // forward state
  size_t delta_b, dq_b, dk_b, dv_b, own2_dk_b, own2_dv_b;  // backward accumulators
  bool split_b, split_h;  // the own backward block runs as two batch halves / head halves
  int b0, h0, nb2, nh2;
  size_t rows2;
};

RingSizes ring_sizes(const ra_shape_t* shape, int nranks) {
  RingSizes z;
  const size_t qrows = (size_t)shape->b * shape->h * shape->lq;
  const size_t krows = (size_t)shape->b * shape->h * shape->lk;
  z.o_bytes = align_up(qrows * shape->dv * 4);
  z.ml_bytes = align_up(qrows * 4);
  z.delta_b = align_up(qrows * 4);
  z.dq_b = align_up(qrows * shape->dk * 4);
  z.dk_b = align_up(krows * shape->dk * 4);
  z.dv_b = align_up(krows * shape->dv * 4);
  // With more than one rank the own block is computed in two parts, the first before and the
  // second after the remote blocks: the second part runs while the last remote block's dK/dV
  // contributions are still travelling and being summed, which would otherwise be exposed.
  // The parts are batch halves, or head halves when there is one batch element; the second
  // part's dK/dV go to a buffer of their own (the owner-side sums write the accumulators
  // meanwhile) and are added at the end.
  z.split_b = nranks > 1 && shape->b >= 2;
  z.split_h = nranks > 1 && shape->b == 1 && shape->h >= 2;
  {
    // the final sum of the second part reads float4: its first row must sit on a 16-byte boundary
    const int64_t off = ((int64_t)(z.split_b ? shape->b / 2 : 0) * shape->h + (z.split_h ? shape->h / 2 : 0)) * shape->lk;
    if ((off * shape->dk) % 4 || (off * shape->dv) % 4) z.split_b = z.split_h = false;
  }
  const bool split = z.split_b || z.split_h;
  z.b0 = z.split_b ? shape->b / 2 : 0;
  z.h0 = z.split_h ? shape->h / 2 : 0;
  z.nb2 = z.split_b ? shape->b - z.b0 : shape->b;
  z.nh2 = z.split_h ? shape->h - z.h0 : shape->h;
  z.rows2 = split ? (size_t)z.nb2 * z.nh2 * shape->lk : 0;
  z.own2_dk_b = align_up(z.rows2 * shape->dk * 4);
  z.own2_dv_b = align_up(z.rows2 * shape->dv * 4);
  return z;
}

// Collective over the ring: all-gathers the IPC handles of this rank's shared buffers and maps
// every peer's.  Runs at creation and whenever the shared buffers have been re-allocated.
// When a rank cannot export or map a buffer (a peer that is not reachable over NVLink / PCIe
// peer access, another node), all ranks agree on it through one more small all-gather and the
// ring falls back to the NCCL transport as a whole: r->p2p becomes false on every rank.
// RA_FAULT_IPC_OPEN=<rank> makes that rank report a failed mapping (host-side fault injection
// for tests).
int exchange_handles(ra_ring_t* r) {
  NcclApi* api = nccl_api();
  IpcBundle mine;
  memset(&mine, 0, sizeof(mine));
  int ok_local = 1;
  for (int i = 0; i < kSlots && ok_local; ++i)
    if (cudaIpcGetMemHandle(&mine.stage[i], r->stage[i]) != cudaSuccess ||
        cudaIpcGetMemHandle(&mine.rpart[i], r->rpart[i]) != cudaSuccess)
      ok_local = 0;
  if (ok_local && cudaIpcGetMemHandle(&mine.flags, r->flags) != cudaSuccess) ok_local = 0;
  if (!ok_local) cudaGetLastError();
  if (const char* inj = getenv("RA_FAULT_IPC_OPEN"))
    if (atoi(inj) == r->rank) ok_local = 0;
  RA_CUDA(cudaMemcpy(r->ipc_send, &mine, sizeof(mine), cudaMemcpyHostToDevice), "cudaMemcpy");
  RA_NCCL(api->AllGather(r->ipc_send, r->ipc_recv, sizeof(mine), ncclChar, r->comm, r->push_stream), "ncclAllGather");
  RA_CUDA(cudaStreamSynchronize(r->push_stream), "cudaStreamSynchronize");
  std::vector<IpcBundle> all(r->nranks);
  RA_CUDA(cudaMemcpy(all.data(), r->ipc_recv, sizeof(mine) * r->nranks, cudaMemcpyDeviceToHost), "cudaMemcpy");
  close_peers(r);
  r->peers.assign(r->nranks, ra_ring::Peer());
  for (int j = 0; j < r->nranks; ++j) {
    ra_ring::Peer& p = r->peers[j];
    if (j == r->rank) {
      for (int i = 0; i < kSlots; ++i) {
        p.stage[i] = r->stage[i];
        p.rpart[i] = r->rpart[i];
      }
      p.flags = r->flags;
      continue;
    }
    if (!ok_local) continue;
    for (int i = 0; i < kSlots && ok_local; ++i)
      if (cudaIpcOpenMemHandle(&p.stage[i], all[j].stage[i], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess ||
          cudaIpcOpenMemHandle(&p.rpart[i], all[j].rpart[i], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
        ok_local = 0;
    void* f = nullptr;
    if (ok_local && cudaIpcOpenMemHandle(&f, all[j].flags, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) ok_local = 0;
    p.flags = (uint64_t*)f;
    if (!ok_local) cudaGetLastError();  // clear the error state: the failure is handled below
  }
  // agree: one failing rank moves the whole ring to the NCCL transport
  RA_CUDA(cudaMemcpy(r->ipc_send, &ok_local, sizeof(int), cudaMemcpyHostToDevice), "cudaMemcpy");
  RA_NCCL(api->AllGather(r->ipc_send, r->ipc_recv, sizeof(int), ncclChar, r->comm, r->push_stream), "ncclAllGather");
  RA_CUDA(cudaStreamSynchronize(r->push_stream), "cudaStreamSynchronize");
  std::vector<int> oks(r->nranks, 0);
  RA_CUDA(cudaMemcpy(oks.data(), r->ipc_recv, sizeof(int) * r->nranks, cudaMemcpyDeviceToHost), "cudaMemcpy");
  bool all_ok = true;
  for (int v : oks) all_ok = all_ok && v != 0;
  if (!all_ok) {
    close_peers(r);
    r->peers.clear();
    r->p2p = false;
  }
  return 0;
}

// Grow-only: (re)allocates the buffers peers write into.  Every rank makes the same calls
// with the same shapes, so every rank grows at the same call and meets in exchange_handles.
int ensure_shared(ra_ring_t* r, size_t stage_need, size_t rpart_need) {
  if (stage_need <= r->stage_bytes && rpart_need <= r->rpart_bytes) return 0;
  RA_CUDA(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  if (r->p2p) close_peers(r);
  const size_t ns = stage_need > r->stage_bytes ? stage_need : r->stage_bytes;
  const size_t np = rpart_need > r->rpart_bytes ? rpart_need : r->rpart_bytes;
  for (int i = 0; i < kSlots; ++i) {
    if (r->stage[i]) cudaFree(r->stage[i]);
    if (r->rpart[i]) cudaFree(r->rpart[i]);
    r->stage[i] = r->rpart[i] = nullptr;
    RA_CUDA(cudaMalloc(&r->stage[i], ns > 0 ? ns : 256), "cudaMalloc(stage)");
    RA_CUDA(cudaMalloc(&r->rpart[i], np > 0 ? np : 256), "cudaMalloc(rpart)");
  }
  r->stage_bytes = ns;
  r->rpart_bytes = np;
  if (r->p2p) return exchange_handles(r);
  return 0;
}

// to / from < 0: that half of the exchange is left out (both ends of it agree, see pair_needed)
RowRuns pair_rows(const ra_ring_t* r, int q_rank, int kv_rank, int lk);

// One side (send or receive) of a K/V message over NCCL: whole parts, or one message per row
// run and batch element.  Both ends derive the same runs from the same plan.
int nccl_part(ra_ring_t* r, const KvMessage& msg, int i, char* base, const RowRuns& rr, int lk, int peer, bool send) {
  NcclApi* api = nccl_api();
  const size_t rb = msg.row_bytes[i];
  auto one = [&](char* p, size_t n) -> int {
    if (send) RA_NCCL(api->Send(p, n, ncclChar, peer, r->comm, r->push_stream), "ncclSend");
    else RA_NCCL(api->Recv(p, n, ncclChar, peer, r->comm, r->push_stream), "ncclRecv");
    return 0;
  };
  if (rb == 0 || (rr.n == 1 && rr.lo[0] == 0 && rr.hi[0] == lk)) return one(base, msg.bytes[i]);
  int rc;
  for (int bb = 0; bb < msg.nb[i]; ++bb)
    for (int k = 0; k < rr.n; ++k)
      if ((rc = one(base + ((size_t)bb * lk + rr.lo[k]) * rb, (size_t)(rr.hi[k] - rr.lo[k]) * rb))) return rc;
  return 0;
}

int exchange_kv_nccl(ra_ring_t* r, const KvMessage& msg, void* stage, int to, int from, int lk) {
  NcclApi* api = nccl_api();
  int rc;
  RA_NCCL(api->GroupStart(), "ncclGroupStart");
  for (int i = 0; i < msg.n; ++i) {
    if (to >= 0 && (rc = nccl_part(r, msg, i, (char*)const_cast<void*>(msg.src[i]), pair_rows(r, to, r->rank, lk), lk, to, true))) return rc;
    if (from >= 0 && (rc = nccl_part(r, msg, i, (char*)stage + msg.offset[i], pair_rows(r, r->rank, from, lk), lk, from, false))) return rc;
  }
  RA_NCCL(api->GroupEnd(), "ncclGroupEnd");
  return 0;
}

// Issue, on the push stream, the transfer that gives the consumer of step t (t >= 1) this
// rank's K/V block.  Called while step t-1 is being enqueued, so it runs under step t-1.
// Under a plan a transfer whose consumer has nothing visible in the block is left out, on both
// sides: sender and receiver read the same matrix.
bool pair_needed(const ra_ring_t* r, int q_rank, int kv_rank) {
  return !r->plan || r->ignore_plan || r->plan->need[(size_t)q_rank * r->nranks + kv_rank] != 0;
}

// The rows of kv_rank's block that the queries of q_rank see something in: whole block without a
// plan (or when the plan was made for another block length).
RowRuns pair_rows(const ra_ring_t* r, int q_rank, int kv_rank, int lk) {
  RowRuns rr;
  rr.hi[0] = lk;
  const ra_ring_plan* pl = r->plan;
  if (!pl || r->ignore_plan || pl->lk != lk || pl->rows.empty()) return rr;
  const int32_t* w = &pl->rows[((size_t)q_rank * r->nranks + kv_rank) * 4];
  rr.n = 0;
  for (int half = 0; half < 2; ++half) {
    int lo = w[half * 2] * 128, hi = w[half * 2 + 1] * 128;
    if (hi > lk) hi = lk;
    if (lo >= hi) continue;
    if (rr.n > 0 && rr.hi[rr.n - 1] == lo) {
      rr.hi[rr.n - 1] = hi;  // the two runs touch: one copy
    } else {
      rr.lo[rr.n] = lo;
      rr.hi[rr.n] = hi;
      ++rr.n;
    }
  }
  return rr;
}

// Copies one part of a K/V message into a peer's staging buffer: whole, or its row runs.
int push_part(ra_ring_t* r, const KvMessage& msg, int i, void* dst_base, const RowRuns& rr, int lk, double* sent) {
  char* dst = (char*)dst_base + msg.offset[i];
  const char* src = (const char*)msg.src[i];
  const size_t rb = msg.row_bytes[i];
  if (rb == 0 || (rr.n == 1 && rr.lo[0] == 0 && rr.hi[0] == lk)) {
    RA_CUDA(cudaMemcpyAsync(dst, src, msg.bytes[i], cudaMemcpyDeviceToDevice, r->push_stream), "cudaMemcpyAsync(peer K/V)");
    *sent += (double)msg.bytes[i];
    return 0;
  }
  const size_t pitch = (size_t)lk * rb;
  for (int k = 0; k < rr.n; ++k) {
    const size_t off = (size_t)rr.lo[k] * rb, width = (size_t)(rr.hi[k] - rr.lo[k]) * rb;
    RA_CUDA(cudaMemcpy2DAsync(dst + off, pitch, src + off, pitch, width, msg.nb[i], cudaMemcpyDeviceToDevice, r->push_stream),
            "cudaMemcpy2DAsync(peer K/V rows)");
    *sent += (double)width * msg.nb[i];
  }
  return 0;
}

int send_kv(ra_ring_t* r, const KvMessage& msg, int t, int lk) {
  const int N = r->nranks, me = r->rank, slot = t % kSlots;
  const int to = (me + t) % N, from = ((me - t) % N + N) % N;
  const bool do_send = pair_needed(r, to, me), do_recv = pair_needed(r, me, from);
  if (r->p2p) {
    if (!do_send) return 0;
    // the consumer's stage[slot] was last read by its step t - kSlots, on the same lane (or by its previous call)
    const uint64_t need = t > kSlots ? r->epoch + t - kSlots + 1 : r->epoch;
    int rc;
    if ((rc = launch_wait(r, r->push_stream, progress_flag(t & 1, to), need))) return rc;
    double sent = 0;
    const RowRuns rr = pair_rows(r, to, me, lk);  // what the consumer's queries see of this rank's block
    if ((rc = push_mark(r, r->push_stream, 0))) return rc;
    for (int i = 0; i < msg.n; ++i)
      if ((rc = push_part(r, msg, i, r->peers[to].stage[slot], rr, lk, &sent))) return rc;
    if ((rc = push_mark(r, r->push_stream, sent))) return rc;
    return launch_set(r, r->push_stream, to, kFlagKvReady + slot, r->epoch + t);
  }
  if (t > kSlots) RA_CUDA(cudaStreamWaitEvent(r->push_stream, r->ev_done[slot], 0), "cudaStreamWaitEvent");
  int rc;
  if ((do_send || do_recv) && (rc = exchange_kv_nccl(r, msg, r->stage[slot], do_send ? to : -1, do_recv ? from : -1, lk))) return rc;
  RA_CUDA(cudaEventRecord(r->ev_recv[slot], r->push_stream), "cudaEventRecord");
  return 0;
}

// Make the compute stream wait until the block of step t (t >= 1) has landed in stage[t & 1].
int wait_kv(ra_ring_t* r, int t, cudaStream_t stream) {
  if (!r->p2p) return wait_transfer(r, stream, r->ev_recv[t % kSlots]);
  int rc;
  if ((rc = timing_mark(r, stream))) return rc;
  if ((rc = launch_wait(r, stream, kFlagKvReady + t % kSlots, r->epoch + t))) return rc;
  return timing_mark(r, stream);
}

// After the block kernel of step t: tell the ranks that may want to overwrite the slot.
int step_done(ra_ring_t* r, int t, cudaStream_t stream) {
  if (r->nranks == 1) return 0;
  RA_CUDA(cudaEventRecord(r->ev_done[t % kSlots], stream), "cudaEventRecord");
  if (!r->p2p) return 0;
  RA_CUDA(cudaStreamWaitEvent(r->flag_stream, r->ev_done[t % kSlots], 0), "cudaStreamWaitEvent");
  return launch_set(r, r->flag_stream, -1, progress_flag(t & 1, r->rank), r->epoch + t + 1);
}

int begin_call(ra_ring_t* ring, int dir, cudaStream_t stream) {
  if (ring->nranks > 1) {
    // transfers read the caller's K/V: order them after whatever produced those
    RA_CUDA(cudaEventRecord(ring->ev_start, stream), "cudaEventRecord");
    RA_CUDA(cudaStreamWaitEvent(ring->push_stream, ring->ev_start, 0), "cudaStreamWaitEvent");
    if (ring->reduce_stream) RA_CUDA(cudaStreamWaitEvent(ring->reduce_stream, ring->ev_start, 0), "cudaStreamWaitEvent");
    RA_CUDA(cudaStreamWaitEvent(ring->lane_stream, ring->ev_start, 0), "cudaStreamWaitEvent");
    RA_CUDA(cudaStreamWaitEvent(ring->give_stream, ring->ev_start, 0), "cudaStreamWaitEvent");
  }
  ring->dir = dir;
  ring->t_used[dir] = 0;
  ring->b_used[dir] = 0;
  ring->p_used[dir] = 0;
  ring->p_bytes[dir] = 0;
  if (ring->timing) RA_CUDA(cudaEventRecord(ring->t_begin[dir], stream), "cudaEventRecord");
  return 0;
}

// The second lane's work of this call is over: move its PROGRESS counter to the call's end and
// make the caller's stream wait for it.
int join_lane(ra_ring_t* ring, cudaStream_t stream) {
  if (ring->nranks == 1) return 0;
  int rc;
  RA_CUDA(cudaEventRecord(ring->ev_lane_done, ring->lane_stream), "cudaEventRecord");
  RA_CUDA(cudaStreamWaitEvent(stream, ring->ev_lane_done, 0), "cudaStreamWaitEvent");
  if (ring->p2p) {
    RA_CUDA(cudaStreamWaitEvent(ring->flag_stream, ring->ev_lane_done, 0), "cudaStreamWaitEvent");
    if ((rc = launch_set(ring, ring->flag_stream, -1, progress_flag(1, ring->rank), ring->epoch + ring->nranks))) return rc;
  }
  return 0;
}

int end_call(ra_ring_t* ring, int dir, cudaStream_t stream) {
  if (ring->nranks > 1) {
    // both lanes' counters end the call at epoch + nranks: the next call's first pushes wait for that
    int rc;
    if (ring->p2p) {
      RA_CUDA(cudaEventRecord(ring->ev_main_end, stream), "cudaEventRecord");
      RA_CUDA(cudaStreamWaitEvent(ring->flag_stream, ring->ev_main_end, 0), "cudaStreamWaitEvent");
      if ((rc = launch_set(ring, ring->flag_stream, -1, progress_flag(0, ring->rank), ring->epoch + ring->nranks))) return rc;
    }
    // the pushes read the caller's tensors: they must be over before the caller may reuse them
    RA_CUDA(cudaEventRecord(ring->ev_push_tail, ring->push_stream), "cudaEventRecord");
    RA_CUDA(cudaStreamWaitEvent(stream, ring->ev_push_tail, 0), "cudaStreamWaitEvent");
    RA_CUDA(cudaEventRecord(ring->ev_give_tail, ring->give_stream), "cudaEventRecord");
    RA_CUDA(cudaStreamWaitEvent(stream, ring->ev_give_tail, 0), "cudaStreamWaitEvent");
    ring->epoch += ring->nranks;
  }
  if (ring->timing) RA_CUDA(cudaEventRecord(ring->t_end[dir], stream), "cudaEventRecord");
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

}  // namespace ringimpl

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
  // The transfer streams get the highest priority: the block kernels fill every SM with one
  // CTA each, and the small kernels that order the transfers must not queue behind them.
  int prio_low = 0, prio_high = 0;
  if ((e = cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high)) != cudaSuccess)
    return bail(fail_cuda(e, "cudaDeviceGetStreamPriorityRange"));
  if ((e = cudaStreamCreateWithPriority(&r->push_stream, cudaStreamNonBlocking, prio_high)) != cudaSuccess ||
      (e = cudaStreamCreateWithPriority(&r->reduce_stream, cudaStreamNonBlocking, prio_high)) != cudaSuccess ||
      (e = cudaStreamCreateWithPriority(&r->lane_stream, cudaStreamNonBlocking, prio_low)) != cudaSuccess ||
      (e = cudaStreamCreateWithPriority(&r->give_stream, cudaStreamNonBlocking, prio_high)) != cudaSuccess ||
      (e = cudaStreamCreateWithPriority(&r->flag_stream, cudaStreamNonBlocking, prio_high)) != cudaSuccess)
    return bail(fail_cuda(e, "cudaStreamCreate"));
  std::vector<cudaEvent_t*> evs = {&r->ev_start, &r->ev_tail, &r->ev_push_tail, &r->ev_step0, &r->ev_lane_start, &r->ev_lane_done,
                                   &r->ev_give_tail, &r->ev_main_end};
  for (int i = 0; i < kSlots; ++i) {
    evs.push_back(&r->ev_recv[i]);
    evs.push_back(&r->ev_done[i]);
    evs.push_back(&r->ev_part[i]);
    evs.push_back(&r->ev_sent[i]);
  }
  for (cudaEvent_t* ev : evs)
    if ((e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming)) != cudaSuccess)
      return bail(fail_cuda(e, "cudaEventCreate"));
  for (int d = 0; d < 2; ++d)
    if ((e = cudaEventCreate(&r->t_begin[d])) != cudaSuccess || (e = cudaEventCreate(&r->t_end[d])) != cudaSuccess)
      return bail(fail_cuda(e, "cudaEventCreate"));
  if ((e = cudaMalloc((void**)&r->guard, 256)) != cudaSuccess || (e = cudaMemset(r->guard, 0, 256)) != cudaSuccess)
    return bail(fail_cuda(e, "cudaMalloc(guard)"));
  {
    const char* env = getenv("RA_RING_WAIT_MS");  // default 10 s
    r->wait_cycles = wait_cycles_of_ms(env ? atoll(env) : 10000);
  }
  if (nranks > 1) {
    if (!nccl_id) return bail(fail(-34, "nccl_id is NULL with nranks > 1"));
    NcclApi* api = nccl_api();
    if (!api) return bail(fail(RA_ERR_NCCL, "NCCL library not found (set RA_NCCL_LIB to libnccl.so.2)"));
    ncclUniqueId uid;
    memcpy(&uid, nccl_id, sizeof(uid));
    ncclResult_t rc = api->CommInitRank(&r->comm, nranks, uid, rank);
    if (rc != ncclSuccess) return bail(fail_nccl(rc, "ncclCommInitRank"));
    const char* tr = getenv("RA_TRANSPORT");
    r->p2p = !(tr && strcmp(tr, "nccl") == 0) && nranks <= kMaxRanks;
    if ((e = cudaMalloc((void**)&r->flags, kNumFlags * sizeof(uint64_t))) != cudaSuccess ||
        (e = cudaMemset(r->flags, 0, kNumFlags * sizeof(uint64_t))) != cudaSuccess ||
        (e = cudaMalloc(&r->ipc_send, sizeof(IpcBundle))) != cudaSuccess ||
        (e = cudaMalloc(&r->ipc_recv, sizeof(IpcBundle) * nranks)) != cudaSuccess ||
        (e = cudaDeviceSynchronize()) != cudaSuccess)
      return bail(fail_cuda(e, "cudaMalloc(flags)"));
    int rc2 = ensure_shared(r, 256, 256);  // maps every peer's flag page (and placeholder buffers)
    if (rc2) return bail(rc2);
  }
  *out = r;
  return 0;
}

int ra_ring_destroy(ra_ring_t* r) {
  if (!r) return 0;
  if (r->push_stream) cudaStreamSynchronize(r->push_stream);
  if (r->reduce_stream) cudaStreamSynchronize(r->reduce_stream);
  if (r->lane_stream) cudaStreamSynchronize(r->lane_stream);
  if (r->give_stream) cudaStreamSynchronize(r->give_stream);
  if (r->flag_stream) cudaStreamSynchronize(r->flag_stream);
  if (r->p2p) close_peers(r);
  if (r->comm) {
    NcclApi* api = nccl_api();
    if (api) api->CommDestroy(r->comm);
  }
  std::vector<cudaEvent_t> evs = {r->ev_start, r->ev_tail, r->ev_push_tail, r->ev_step0, r->ev_lane_start, r->ev_lane_done,
                                  r->ev_give_tail, r->ev_main_end, r->t_begin[0], r->t_begin[1], r->t_end[0], r->t_end[1]};
  for (int i = 0; i < kSlots; ++i) {
    evs.push_back(r->ev_recv[i]);
    evs.push_back(r->ev_done[i]);
    evs.push_back(r->ev_part[i]);
    evs.push_back(r->ev_sent[i]);
  }
  for (cudaEvent_t ev : evs)
    if (ev) cudaEventDestroy(ev);
  for (int d = 0; d < 2; ++d) {
    for (cudaEvent_t ev : r->t_events[d]) cudaEventDestroy(ev);
    for (cudaEvent_t ev : r->b_events[d]) cudaEventDestroy(ev);
    for (cudaEvent_t ev : r->p_events[d]) cudaEventDestroy(ev);
  }
  if (r->push_stream) cudaStreamDestroy(r->push_stream);
  if (r->reduce_stream) cudaStreamDestroy(r->reduce_stream);
  if (r->lane_stream) cudaStreamDestroy(r->lane_stream);
  if (r->give_stream) cudaStreamDestroy(r->give_stream);
  if (r->flag_stream) cudaStreamDestroy(r->flag_stream);
  r->state.release();
  r->grads.release();
  for (int i = 0; i < kSlots; ++i) {
    r->part[i].release();
    if (r->stage[i]) cudaFree(r->stage[i]);
    if (r->rpart[i]) cudaFree(r->rpart[i]);
  }
  if (r->flags) cudaFree(r->flags);
  if (r->guard) cudaFree(r->guard);
  if (r->ipc_send) cudaFree(r->ipc_send);
  if (r->ipc_recv) cudaFree(r->ipc_recv);
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

int ra_ring_set_wait_ms(ra_ring_t* r, int32_t ms) {
  if (!r) return fail(-30, "ring handle is NULL");
  if (ms < 1) return fail(-43, "the wait bound must be at least 1 ms");
  r->wait_cycles = wait_cycles_of_ms(ms);
  return 0;
}

int ra_ring_probe_wait(ra_ring_t* r, void* stream) {
  if (!r) return fail(-30, "ring handle is NULL");
  unsigned int* status = device_status_word();
  if (!status) return fail(RA_ERR_CUDA, "status word symbol not found");
  // guard[2..3]: a counter that stays 0 for the life of the ring; the target is never reached
  wait_flag_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(reinterpret_cast<const uint64_t*>(r->guard + 2), 1, status, r->guard,
                                                     r->wait_cycles);
  count_launch();
  RA_CUDA(cudaGetLastError(), "wait_flag_kernel");
  return 0;
}

int ra_ring_aborted(ra_ring_t* r) {
  if (!r) return fail(-30, "ring handle is NULL");
  unsigned int v = 0;
  RA_CUDA(cudaMemcpy(&v, r->guard, sizeof(v), cudaMemcpyDeviceToHost), "cudaMemcpy");
  return v ? 1 : 0;
}

int ra_ring_transport(const ra_ring_t* r) {
  if (!r) return fail(-30, "ring handle is NULL");
  return r->nranks == 1 ? 0 : (r->p2p ? 1 : 2);
}

namespace ringimpl {
// [begin, end) offsets in ms from the call's first event, one interval per pair of events.
int event_intervals(cudaEvent_t origin, const std::vector<cudaEvent_t>& ev, size_t used,
                    std::vector<std::pair<float, float>>* out) {
  out->clear();
  for (size_t i = 0; i + 1 < used; i += 2) {
    float a = 0.f, b = 0.f;
    RA_CUDA(cudaEventElapsedTime(&a, origin, ev[i]), "cudaEventElapsedTime");
    RA_CUDA(cudaEventElapsedTime(&b, origin, ev[i + 1]), "cudaEventElapsedTime");
    out->push_back({a, b > a ? b : a});
  }
  return 0;
}

// Sorted, disjoint union of intervals.
std::vector<std::pair<float, float>> interval_union(std::vector<std::pair<float, float>> v) {
  std::sort(v.begin(), v.end());
  std::vector<std::pair<float, float>> u;
  for (const auto& iv : v) {
    if (!u.empty() && iv.first <= u.back().second)
      u.back().second = std::max(u.back().second, iv.second);
    else
      u.push_back(iv);
  }
  return u;
}
}  // namespace ringimpl

// Exposed wait = the part of each wait for a transfer during which no block kernel of this
// rank was running (with two compute lanes a wait on one lane is hidden while the other lane
// computes).
int ra_ring_last_timing(ra_ring_t* r, int32_t backward, float* total_ms, float* exposed_ms) {
  if (!r) return fail(-30, "ring handle is NULL");
  if (!r->timing) return fail(-35, "timing is off: call ra_ring_set_timing(ring, 1) first");
  const int d = backward ? 1 : 0;
  RA_CUDA(cudaEventSynchronize(r->t_end[d]), "cudaEventSynchronize");
  float tot = 0.f, exp = 0.f;
  RA_CUDA(cudaEventElapsedTime(&tot, r->t_begin[d], r->t_end[d]), "cudaEventElapsedTime");
  std::vector<std::pair<float, float>> waits, blocks;
  int rc;
  if ((rc = event_intervals(r->t_begin[d], r->t_events[d], r->t_used[d], &waits))) return rc;
  if ((rc = event_intervals(r->t_begin[d], r->b_events[d], r->b_used[d], &blocks))) return rc;
  const auto busy = interval_union(blocks);
  for (const auto& w : waits) {
    float hidden = 0.f;
    for (const auto& k : busy) {
      const float lo = std::max(w.first, k.first), hi = std::min(w.second, k.second);
      if (hi > lo) hidden += hi - lo;
    }
    exp += (w.second - w.first) - hidden;
  }
  if (total_ms) *total_ms = tot;
  if (exposed_ms) *exposed_ms = exp;
  return 0;
}

int ra_ring_last_timeline(ra_ring_t* r, int32_t backward, int32_t max_items, float* blocks, int32_t* n_blocks,
                          float* waits, int32_t* n_waits) {
  if (!r) return fail(-30, "ring handle is NULL");
  if (!r->timing) return fail(-35, "timing is off: call ra_ring_set_timing(ring, 1) first");
  if (max_items < 0 || !blocks || !waits || !n_blocks || !n_waits) return fail(-6, "timeline: result pointers are NULL");
  const int d = backward ? 1 : 0;
  RA_CUDA(cudaEventSynchronize(r->t_end[d]), "cudaEventSynchronize");
  std::vector<std::pair<float, float>> w, b;
  int rc;
  if ((rc = event_intervals(r->t_begin[d], r->t_events[d], r->t_used[d], &w))) return rc;
  if ((rc = event_intervals(r->t_begin[d], r->b_events[d], r->b_used[d], &b))) return rc;
  *n_blocks = (int32_t)std::min<size_t>(b.size(), (size_t)max_items);
  *n_waits = (int32_t)std::min<size_t>(w.size(), (size_t)max_items);
  for (int i = 0; i < *n_blocks; ++i) blocks[2 * i] = b[i].first, blocks[2 * i + 1] = b[i].second;
  for (int i = 0; i < *n_waits; ++i) waits[2 * i] = w[i].first, waits[2 * i + 1] = w[i].second;
  return 0;
}

int ra_ring_last_push(ra_ring_t* r, int32_t backward, double* bytes, float* push_ms) {
  if (!r) return fail(-30, "ring handle is NULL");
  if (!r->timing) return fail(-35, "timing is off: call ra_ring_set_timing(ring, 1) first");
  const int dir = backward ? 1 : 0;
  RA_CUDA(cudaEventSynchronize(r->t_end[dir]), "cudaEventSynchronize");
  if (r->push_stream) RA_CUDA(cudaStreamSynchronize(r->push_stream), "cudaStreamSynchronize");
  if (r->give_stream) RA_CUDA(cudaStreamSynchronize(r->give_stream), "cudaStreamSynchronize");
  float sum = 0.f;
  for (size_t i = 0; i + 1 < r->p_used[dir]; i += 2) {
    float ms = 0.f;
    RA_CUDA(cudaEventElapsedTime(&ms, r->p_events[dir][i], r->p_events[dir][i + 1]), "cudaEventElapsedTime");
    sum += ms;
  }
  if (bytes) *bytes = r->p_bytes[dir];
  if (push_ms) *push_ms = sum;
  return 0;
}

int ra_ring_last_block_ms(ra_ring_t* r, int32_t backward, float* block_ms, int32_t* launches) {
  if (!r) return fail(-30, "ring handle is NULL");
  if (!r->timing) return fail(-35, "timing is off: call ra_ring_set_timing(ring, 1) first");
  const int dir = backward ? 1 : 0;
  if (r->b_used[dir] == 0) return fail(-38, "no %s call has been timed yet", dir ? "backward" : "forward");
  RA_CUDA(cudaEventSynchronize(r->t_end[dir]), "cudaEventSynchronize");
  // device time during which at least one block kernel ran (kernels of the two lanes overlap)
  std::vector<std::pair<float, float>> blocks;
  int rc;
  if ((rc = event_intervals(r->t_begin[dir], r->b_events[dir], r->b_used[dir], &blocks))) return rc;
  float sum = 0.f;
  for (const auto& k : interval_union(blocks)) sum += k.second - k.first;
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
  const int N = ring->nranks;
  p.b = shape->b;
  p.h = shape->h;
  p.lq = shape->lq;
  p.lk = shape->lk;
  p.dk = shape->dk;
  p.dv = shape->dv;
  p.scale = shape->sm_scale;

  const RingSizes z = ring_sizes(shape, N);
  const size_t o_bytes = z.o_bytes, ml_bytes = z.ml_bytes, state_bytes = o_bytes + 2 * ml_bytes;
  // one carried state (o, m, l) per compute lane: even steps fold into the first, odd steps into
  // the second, and the two are merged at the end (the online-softmax update of ring.py:58-76 is
  // associative), so that adjacent steps do not depend on each other
  const int n_lanes = N > 1 ? 2 : 1;
  RA_CUDA(ring->state.reserve(n_lanes * state_bytes), "cudaMalloc(state)");
  float *st_o[2], *st_m[2], *st_l[2];
  for (int ln = 0; ln < 2; ++ln) {
    char* base = (char*)ring->state.ptr + (ln < n_lanes ? ln : 0) * state_bytes;
    st_o[ln] = (float*)base;
    st_m[ln] = (float*)(base + o_bytes);
    st_l[ln] = (float*)(base + o_bytes + ml_bytes);
  }
  cudaStream_t lane_s[2] = {stream, N > 1 ? ring->lane_stream : stream};

  ring->ignore_plan = (p.mod.kinds & RA_MOD_STRICT_NAN) != 0;
  KvMessage msg = make_kv_message(shape, p.k, p.v, p.mod);
  if (N > 1 && (rc = ensure_shared(ring, msg.total, 0))) return rc;
  if ((rc = begin_call(ring, 0, stream))) return rc;

  const TensorView k_own = p.k, v_own = p.v;
  const ModParams mod_own = p.mod;
  const TensorView out_view{out->ptr, out->stride_b, out->stride_l, out->stride_h};
  if (ring->plan && ring->plan->nranks != N) return fail(-39, "the plan was made for a ring of %d ranks", ring->plan->nranks);
  const int me_f = ring->rank;
  auto source = [&](int t) { return ((me_f - t) % N + N) % N; };
  bool used[2] = {false, false};
  for (int t = 0; t < N; ++t) {
    const int ln = t & (n_lanes - 1);
    cudaStream_t s = lane_s[ln];
    if (t + 1 < N && (rc = send_kv(ring, msg, t + 1, shape->lk))) return rc;  // runs under step t
    if (t > 0 && !pair_needed(ring, me_f, source(t))) {  // nothing visible in this block: no wait, no launch
      if ((rc = step_done(ring, t, s))) return rc;
      continue;
    }
    p.k = k_own;
    p.v = v_own;
    p.mod = mod_own;
    p.o = st_o[ln];
    p.m = st_m[ln];
    p.l = st_l[ln];
    if (t > 0) {
      use_staged(msg, ring->stage[t % kSlots], &p.k, &p.v, &p.mod);
      if ((rc = wait_kv(ring, t, s))) return rc;
    }
    p.first = !used[ln];
    used[ln] = true;
    if (N == 1) {  // ring of one: the tensor-core kernel normalises and writes out / L itself
      p.final_out = out_view;
      p.final_lse = lse;
    }
    if ((rc = block_mark(ring, 0, s))) return rc;
    if ((rc = run_fwd_block(p, shape->dtype, s))) return rc;
    if ((rc = block_mark(ring, 0, s))) return rc;
    if ((rc = step_done(ring, t, s))) return rc;
  }
  if ((rc = join_lane(ring, stream))) return rc;
  if (N > 1 || last_impl() != RA_IMPL_TCGEN05) {  // ring.py:134-135 over the merged states of the lanes
    cudaError_t e = launch_finalize(shape->b, shape->h, shape->lq, shape->dv, st_o[0], st_m[0], st_l[0],
                                    used[1] ? st_o[1] : nullptr, st_m[1], st_l[1], out_view, shape->dtype, lse, stream);
    if (e != cudaSuccess) return fail_cuda(e, "finalize");
  }
  // no contributions were exchanged in this call: move this rank's ADDED counter to the call's end
  if (N > 1 && ring->p2p && (rc = launch_set(ring, stream, -1, kFlagAdded + ring->rank, ring->epoch + N))) return rc;
  return end_call(ring, 0, stream);
}

namespace ringimpl {
// The part of a backward block call that covers batch elements [b0, b0 + nb) and heads
// [h0, h0 + nh) (a head range only with one batch element: the fp32 state arrays are
// [b, h, len, d] and must stay dense).  Everything is a pointer offset; shapes shrink.
BwdParams sub_problem(const BwdParams& p, int esize, int b0, int nb, int h0, int nh) {
  BwdParams s = p;
  auto view = [&](TensorView t) {
    if (t.ptr) t.ptr = (const char*)t.ptr + ((int64_t)b0 * t.sb + (int64_t)h0 * t.sh) * esize;
    return t;
  };
  s.q = view(p.q);
  s.k = view(p.k);
  s.v = view(p.v);
  s.dout = view(p.dout);
  if (s.mod.q_pos) s.mod.q_pos += (int64_t)b0 * p.lq;
  if (s.mod.q_seg) s.mod.q_seg += (int64_t)b0 * p.lq;
  if (s.mod.q_pre) s.mod.q_pre += (int64_t)b0 * p.lq;
  if (s.mod.kv_pos) s.mod.kv_pos += (int64_t)b0 * p.lk;
  if (s.mod.kv_seg) s.mod.kv_seg += (int64_t)b0 * p.lk;
  if (s.mod.kv_pre) s.mod.kv_pre += (int64_t)b0 * p.lk;
  if (s.mod.slopes) s.mod.slopes += h0;
  const int64_t bh0 = (int64_t)b0 * p.h + h0;
  s.lse = p.lse + bh0 * p.lq;
  s.delta = p.delta + bh0 * p.lq;
  if (p.row_nl2) s.row_nl2 = p.row_nl2 + bh0 * p.lq;
  if (p.row_nds) s.row_nds = p.row_nds + bh0 * p.lq;
  s.dq = p.dq + bh0 * p.lq * p.dk_dim;
  s.dk = p.dk + bh0 * p.lk * p.dk_dim;
  s.dv = p.dv + bh0 * p.lk * p.dv_dim;
  s.b = nb;
  s.h = nh;
  return s;
}
}  // namespace ringimpl

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

  const RingSizes z = ring_sizes(shape, N);
  const size_t delta_b = z.delta_b, dq_b = z.dq_b, dk_b = z.dk_b, dv_b = z.dv_b;
  const int esize = shape->dtype == RA_DTYPE_BF16 ? 2 : 4;
  const bool split_b = z.split_b, split_h = z.split_h, split = split_b || split_h;
  const int b0 = z.b0, h0 = z.h0, nb2 = z.nb2, nh2 = z.nh2;
  const size_t rows2 = z.rows2, own2_dk_b = z.own2_dk_b, own2_dv_b = z.own2_dv_b;
  // delta, then the two per-row terms derived from L and delta that the tensor-core kernel reads
  RA_CUDA(ring->grads.reserve(3 * delta_b + dq_b + dk_b + dv_b + own2_dk_b + own2_dv_b), "cudaMalloc(grads)");
  char* g = (char*)ring->grads.ptr + 2 * delta_b;
  float* row_nl2 = (float*)ring->grads.ptr;
  float* row_nds = (float*)((char*)ring->grads.ptr + delta_b);
  float* delta = (float*)g;
  float* dq_acc = (float*)(g + delta_b);
  float* dk_acc = (float*)(g + delta_b + dq_b);
  float* dv_acc = (float*)(g + delta_b + dq_b + dk_b);
  float* own2_dk = (float*)(g + delta_b + dq_b + dk_b + dv_b);
  float* own2_dv = (float*)(g + delta_b + dq_b + dk_b + dv_b + own2_dk_b);
  KvMessage msg = make_kv_message(shape, p.k, p.v, p.mod);
  if (N > 1) {
    for (int i = 0; i < kSlots; ++i) RA_CUDA(ring->part[i].reserve(dk_b + dv_b), "cudaMalloc(part)");
    if ((rc = ensure_shared(ring, msg.total, dk_b + dv_b))) return rc;
  }
  if (ring->plan && ring->plan->nranks != ring->nranks)
    return fail(-39, "the plan was made for a ring of %d ranks", ring->plan->nranks);
  if ((rc = begin_call(ring, 1, stream))) return rc;

  cudaError_t e = launch_delta(shape->b, shape->h, shape->lq, shape->dv, tv(out), p.dout,
                               shape->dtype, delta, stream);
  if (e != cudaSuccess) return fail_cuda(e, "delta");
  p.delta = delta;
  if (current_impl() != RA_IMPL_SIMT) {  // once per backward, not once per block launch
    e = launch_bwd_row_terms(lse, delta, shape->sm_scale, 1, (int64_t)shape->b * shape->h * shape->lq, row_nl2, row_nds, stream);
    if (e != cudaSuccess) return fail_cuda(e, "row terms");
    p.row_nl2 = row_nl2;
    p.row_nds = row_nds;
  }
  p.dq = dq_acc;
  // Ring of one on the tensor-core path: the kernel stores dK, dV in the result dtype itself, so
  // their fp32 accumulators are neither cleared nor converted.
  p.dk = dk_acc;
  p.dv = dv_acc;
  bool direct = false;
  ring->ignore_plan = (p.mod.kinds & RA_MOD_STRICT_NAN) != 0;
  if (N == 1 && current_impl() != RA_IMPL_SIMT && !(p.mod.kinds & RA_MOD_STRICT_NAN)) {
    p.dk_out = tv(dk);
    p.dv_out = tv(dv);
    direct = tc_bwd_unsupported_reason(p, shape->dtype) == nullptr;
    if (!direct) p.dk_out = p.dv_out = TensorView{nullptr, 0, 0, 0};
  }
  RA_CUDA(cudaMemsetAsync(dq_acc, 0, direct ? dq_b : dq_b + dk_b + dv_b, stream), "cudaMemsetAsync");
  count_launch();
  if (direct) {
    if ((rc = block_mark(ring, 1, stream))) return rc;
    e = tc_bwd_block(p, stream);
    if (e == cudaSuccess) {
      set_last_impl(RA_IMPL_TCGEN05);
      if ((rc = block_mark(ring, 1, stream))) return rc;
      if ((e = launch_cast_from_f32(shape->b, shape->h, shape->lq, shape->dk, dq_acc, tv(dq), shape->dtype, stream)) != cudaSuccess)
        return fail_cuda(e, "cast");
      return end_call(ring, 1, stream);
    }
    if (e != cudaErrorNotSupported) return fail_cuda(e, "tcgen05 backward block");
    // the driver refused a tensor map: take the general path below
    ring->b_used[1] = 0;
    p.dk_out = p.dv_out = TensorView{nullptr, 0, 0, 0};
    RA_CUDA(cudaMemsetAsync(dk_acc, 0, dk_b + dv_b, stream), "cudaMemsetAsync");
  }

  NcclApi* api = N > 1 ? nccl_api() : nullptr;
  cudaStream_t add_stream = ring->p2p ? ring->reduce_stream : ring->push_stream;
  // even steps on the caller's stream, odd steps on the second compute lane: adjacent block
  // kernels share nothing but the dQ accumulator (added to with reductions), so the tail of one
  // overlaps the head of the next
  cudaStream_t lane_s[2] = {stream, N > 1 ? ring->lane_stream : stream};
  if (N > 1) {  // delta is computed and the accumulators are cleared
    RA_CUDA(cudaEventRecord(ring->ev_lane_start, stream), "cudaEventRecord");
    RA_CUDA(cudaStreamWaitEvent(ring->lane_stream, ring->ev_lane_start, 0), "cudaStreamWaitEvent");
  }
  const TensorView k_own = p.k, v_own = p.v;
  const ModParams mod_own = p.mod;
  for (int t = 0; t < N; ++t) {
    cudaStream_t s = lane_s[t & 1];
    if (t + 1 < N && (rc = send_kv(ring, msg, t + 1, shape->lk))) return rc;
    p.k = k_own;
    p.v = v_own;
    p.mod = mod_own;
    if (t == 0) {
      p.dk = dk_acc;
      p.dv = dv_acc;
      const BwdParams first = split ? sub_problem(p, esize, 0, split_b ? b0 : shape->b, 0, split_h ? h0 : shape->h) : p;
      if ((rc = block_mark(ring, 1, s))) return rc;
      if ((rc = run_bwd_block(first, shape->dtype, s))) return rc;
      if ((rc = block_mark(ring, 1, s))) return rc;
      if ((rc = step_done(ring, 0, s))) return rc;
      if (N > 1) {  // the sums of received contributions start after the accumulators were cleared and the own block's part added
        RA_CUDA(cudaEventRecord(ring->ev_step0, s), "cudaEventRecord");
        if (ring->p2p) RA_CUDA(cudaStreamWaitEvent(ring->reduce_stream, ring->ev_step0, 0), "cudaStreamWaitEvent");
      }
      continue;
    }
    const int slot = t % kSlots;
    const int owner = ((me - t) % N + N) % N, giver = (me + t) % N;
    // Under a plan: this rank computes (and gives) only where its queries see the block, and
    // receives only where the giver's queries see this rank's block.
    const bool compute = pair_needed(ring, me, owner), receive = pair_needed(ring, giver, me);
    // key rows of the contribution this rank gives (those its queries saw in the owner's block)
    // and of the one it receives (those the giver's queries saw in this rank's block)
    const RowRuns give_rows = pair_rows(ring, me, owner, shape->lk), take_rows = pair_rows(ring, giver, me, shape->lk);
    auto whole = [&](const RowRuns& rr) { return rr.n == 1 && rr.lo[0] == 0 && rr.hi[0] == shape->lk; };
    if (compute) {
      use_staged(msg, ring->stage[slot], &p.k, &p.v, &p.mod);
      if ((rc = wait_kv(ring, t, s))) return rc;
      // part[slot] was last sent kSlots steps ago
      if (t > kSlots) RA_CUDA(cudaStreamWaitEvent(s, ring->ev_sent[slot], 0), "cudaStreamWaitEvent");
      // this step's contribution is built from nothing: the kernel stores instead of adding
      p.dk = (float*)ring->part[slot].ptr;
      p.dv = (float*)((char*)ring->part[slot].ptr + dk_b);
      p.overwrite = 1;
      if ((rc = block_mark(ring, 1, s))) return rc;
      if ((rc = run_bwd_block(p, shape->dtype, s))) return rc;
      if ((rc = block_mark(ring, 1, s))) return rc;
      p.overwrite = 0;
    }
    if ((rc = step_done(ring, t, s))) return rc;
    // the stream this step's contribution travels on
    cudaStream_t xfer = ring->p2p ? ring->give_stream : ring->push_stream;
    if (compute) {
      RA_CUDA(cudaEventRecord(ring->ev_part[slot], s), "cudaEventRecord");
      // give it to the block's owner; take what another rank computed for this rank's block
      RA_CUDA(cudaStreamWaitEvent(xfer, ring->ev_part[slot], 0), "cudaStreamWaitEvent");
    }
    if (ring->p2p) {
      if (compute) {
        // the owner's rpart[slot] is free once it has summed the contribution of step t - kSlots
        const uint64_t need = t > kSlots ? ring->epoch + t - kSlots + 1 : ring->epoch;
        if ((rc = launch_wait(ring, xfer, kFlagAdded + owner, need))) return rc;
        if ((rc = push_mark(ring, xfer, 0))) return rc;
        double sent = 0;
        if (whole(give_rows)) {
          RA_CUDA(cudaMemcpyAsync(ring->peers[owner].rpart[slot], ring->part[slot].ptr, dk_b + dv_b,
                                  cudaMemcpyDeviceToDevice, xfer), "cudaMemcpyAsync(peer dK/dV)");
          sent = (double)(dk_b + dv_b);
        } else {  // only the key rows this rank's queries saw: one strided copy per run, dK and dV
          for (int k = 0; k < give_rows.n; ++k)
            for (int which = 0; which < 2; ++which) {
              const size_t d = which ? shape->dv : shape->dk, base = which ? dk_b : 0;
              const size_t pitch = (size_t)shape->lk * d * 4, off = base + (size_t)give_rows.lo[k] * d * 4;
              const size_t width = (size_t)(give_rows.hi[k] - give_rows.lo[k]) * d * 4;
              RA_CUDA(cudaMemcpy2DAsync((char*)ring->peers[owner].rpart[slot] + off, pitch, (char*)ring->part[slot].ptr + off, pitch,
                                        width, (size_t)shape->b * shape->h, cudaMemcpyDeviceToDevice, xfer),
                      "cudaMemcpy2DAsync(peer dK/dV rows)");
              sent += (double)width * shape->b * shape->h;
            }
        }
        if ((rc = push_mark(ring, xfer, sent))) return rc;
        if ((rc = launch_set(ring, xfer, owner, kFlagPartReady + slot, ring->epoch + t))) return rc;
        RA_CUDA(cudaEventRecord(ring->ev_sent[slot], xfer), "cudaEventRecord");
      }
      // owner side, on the reduce stream
      if (receive && (rc = launch_wait(ring, ring->reduce_stream, kFlagPartReady + slot, ring->epoch + t))) return rc;
    } else if (compute || receive) {
      // whole buffers, or one message per (batch, head) and row run of dK and of dV
      auto nccl_rows = [&](char* base, const RowRuns& rr, int peer, bool send) -> int {
        auto one = [&](char* ptr, size_t n) -> int {
          if (send) RA_NCCL(api->Send(ptr, n, ncclChar, peer, ring->comm, ring->push_stream), "ncclSend");
          else RA_NCCL(api->Recv(ptr, n, ncclChar, peer, ring->comm, ring->push_stream), "ncclRecv");
          return 0;
        };
        if (whole(rr)) return one(base, dk_b + dv_b);
        int rc2;
        for (int which = 0; which < 2; ++which) {
          const size_t d = which ? shape->dv : shape->dk, off0 = which ? dk_b : 0;
          for (int64_t seg = 0; seg < (int64_t)shape->b * shape->h; ++seg)
            for (int k = 0; k < rr.n; ++k)
              if ((rc2 = one(base + off0 + ((size_t)seg * shape->lk + rr.lo[k]) * d * 4, (size_t)(rr.hi[k] - rr.lo[k]) * d * 4))) return rc2;
        }
        return 0;
      };
      RA_NCCL(api->GroupStart(), "ncclGroupStart");
      if (compute && (rc = nccl_rows((char*)ring->part[slot].ptr, give_rows, owner, true))) return rc;
      if (receive && (rc = nccl_rows((char*)ring->rpart[slot], take_rows, giver, false))) return rc;
      RA_NCCL(api->GroupEnd(), "ncclGroupEnd");
      RA_CUDA(cudaEventRecord(ring->ev_sent[slot], ring->push_stream), "cudaEventRecord");
    }
    if (receive) {
      // NCCL transport: the sum runs on the transfer stream, which has not seen the own block yet
      if (!ring->p2p) RA_CUDA(cudaStreamWaitEvent(add_stream, ring->ev_step0, 0), "cudaStreamWaitEvent");
      if (whole(take_rows)) {
        e = launch_add_f32(dk_acc, (const float*)ring->rpart[slot], (int64_t)((dk_b + dv_b) / 4), add_stream);
      } else {
        e = cudaSuccess;
        for (int k = 0; k < take_rows.n && e == cudaSuccess; ++k)
          for (int which = 0; which < 2 && e == cudaSuccess; ++which) {
            const int64_t d = which ? shape->dv : shape->dk;
            float* dst = which ? dv_acc : dk_acc;
            const float* src = (const float*)((const char*)ring->rpart[slot] + (which ? dk_b : 0));
            e = launch_add_rows_f32(dst + take_rows.lo[k] * d, src + take_rows.lo[k] * d, (int64_t)shape->b * shape->h,
                                    (int64_t)(take_rows.hi[k] - take_rows.lo[k]) * d, (int64_t)shape->lk * d, add_stream);
          }
      }
      if (e != cudaSuccess) return fail_cuda(e, "add");
    }
    // published even when nothing was received: it is what frees rpart[slot] for the step after next
    if (ring->p2p && (rc = launch_set(ring, ring->reduce_stream, -1, kFlagAdded + me, ring->epoch + t + 1))) return rc;
  }
  if (N > 1) RA_CUDA(cudaEventRecord(ring->ev_tail, add_stream), "cudaEventRecord");
  if (split) {
    // on the lane of the last remote step, behind it: that step's contribution then travels and
    // is summed while this part runs (on the other lane the two kernels would share the GPU and
    // end together, with the transfer exposed after them)
    cudaStream_t s = lane_s[(N - 1) & 1];
    p.k = k_own;
    p.v = v_own;
    p.mod = mod_own;
    p.dk = dk_acc;
    p.dv = dv_acc;
    BwdParams second = sub_problem(p, esize, b0, nb2, h0, nh2);
    second.dk = own2_dk;
    second.dv = own2_dv;
    second.overwrite = 1;  // built from nothing: no clearing pass
    if ((rc = block_mark(ring, 1, s))) return rc;
    if ((rc = run_bwd_block(second, shape->dtype, s))) return rc;
    if ((rc = block_mark(ring, 1, s))) return rc;
  }
  if ((rc = join_lane(ring, stream))) return rc;
  if (N > 1 && (rc = wait_transfer(ring, stream, ring->ev_tail))) return rc;
  if (split) {
    const int64_t off = ((int64_t)b0 * shape->h + h0) * shape->lk;
    if ((e = launch_add_f32(dk_acc + off * shape->dk, own2_dk, (int64_t)rows2 * shape->dk, stream)) != cudaSuccess ||
        (e = launch_add_f32(dv_acc + off * shape->dv, own2_dv, (int64_t)rows2 * shape->dv, stream)) != cudaSuccess)
      return fail_cuda(e, "add");
  }
  if ((e = launch_cast_from_f32(shape->b, shape->h, shape->lq, shape->dk, dq_acc, tv(dq), shape->dtype, stream)) != cudaSuccess ||
      (e = launch_cast_from_f32(shape->b, shape->h, shape->lk, shape->dk, dk_acc, tv(dk), shape->dtype, stream)) != cudaSuccess ||
      (e = launch_cast_from_f32(shape->b, shape->h, shape->lk, shape->dv, dv_acc, tv(dv), shape->dtype, stream)) != cudaSuccess)
    return fail_cuda(e, "cast");
  return end_call(ring, 1, stream);
}

int ra_ring_reserve(ra_ring_t* ring, const ra_shape_t* shape, const ra_score_mod_t* mod, int32_t backward) {
  int rc;
  if (!ring) return fail(-30, "ring handle is NULL");
  if ((rc = check_shape(shape))) return rc;
  int dev = -1;
  RA_CUDA(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev != ring->device) return fail(-31, "ring was created on device %d but device %d is current", ring->device, dev);
  const int N = ring->nranks;
  const RingSizes z = ring_sizes(shape, N);
  // size of one K/V block message: only which per-token arrays exist matters, not where they are
  ModParams m;
  memset(&m, 0, sizeof(m));
  if (mod) {
    m.kv_pos = mod->kv_pos;
    m.kv_seg = mod->kv_seg;
    m.kv_pre = mod->kv_prefix;
  }
  const TensorView none{nullptr, 0, 0, 0};
  const KvMessage msg = make_kv_message(shape, none, none, m);
  RA_CUDA(ring->state.reserve(z.o_bytes + 2 * z.ml_bytes), "cudaMalloc(state)");
  if (backward) {
    RA_CUDA(ring->grads.reserve(3 * z.delta_b + z.dq_b + z.dk_b + z.dv_b + z.own2_dk_b + z.own2_dv_b), "cudaMalloc(grads)");
    if (N > 1)
      for (int i = 0; i < kSlots; ++i) RA_CUDA(ring->part[i].reserve(z.dk_b + z.dv_b), "cudaMalloc(part)");
  }
  if (N > 1 && (rc = ensure_shared(ring, msg.total, backward ? z.dk_b + z.dv_b : 0))) return rc;
  // the block kernels take their tile summaries from a stream-ordered pool that keeps what it
  // was given: give it this shape's worth now
  void* tmp = nullptr;
  const size_t meta_bytes = (size_t)shape->b * ((shape->lq + 127) / 128 + (shape->lk + 127) / 128) * sizeof(TileMeta);
  RA_CUDA(scratch_alloc(&tmp, meta_bytes, ring->push_stream), "scratch pool");
  RA_CUDA(cudaFreeAsync(tmp, ring->push_stream), "cudaFreeAsync");
  RA_CUDA(cudaStreamSynchronize(ring->push_stream), "cudaStreamSynchronize");
  return 0;
}

int ra_ring_plan_create(ra_ring_t* ring, const ra_shape_t* shape, const ra_score_mod_t* mod, void* stream_,
                        ra_ring_plan_t** out) {
  int rc;
  if (!ring) return fail(-30, "ring handle is NULL");
  if (!out) return fail(-6, "plan result pointer is NULL");
  *out = nullptr;
  if ((rc = check_shape(shape))) return rc;
  ModParams m;
  if ((rc = check_mod(mod, &m))) return rc;
  const int N = ring->nranks;
  ra_ring_plan* plan = new ra_ring_plan;
  plan->nranks = N;
  plan->need.assign((size_t)N * N, 1);
  // without a mask every pair has visible pairs; a dense bias tile cannot be summarised
  if (N == 1 || !(m.kinds & kMaskKinds) || (m.kinds & RA_MOD_DENSE)) {
    *out = plan;
    return 0;
  }
  cudaStream_t s = (cudaStream_t)stream_;
  const int b = shape->b, nq = (shape->lq + 127) / 128, nk = (shape->lk + 127) / 128;
  const size_t per_rank = (size_t)b * (nq + nk);
  TileMeta *mine = nullptr, *all = nullptr;
  int* need_dev = nullptr;  // [N * N] need flags, then [N * N * 4] row runs
  std::vector<int> need_host((size_t)N * N * 5, 1);
  auto cleanup = [&]() {
    if (mine) cudaFree(mine);
    if (all) cudaFree(all);
    if (need_dev) cudaFree(need_dev);
  };
  auto bail = [&](int code) {
    cleanup();
    delete plan;
    return code;
  };
  cudaError_t e;
  if ((e = cudaMalloc((void**)&mine, per_rank * sizeof(TileMeta))) != cudaSuccess ||
      (e = cudaMalloc((void**)&all, per_rank * sizeof(TileMeta) * N)) != cudaSuccess ||
      (e = cudaMalloc((void**)&need_dev, sizeof(int) * N * N * 5)) != cudaSuccess)
    return bail(fail_cuda(e, "cudaMalloc(plan)"));
  plan_meta_kernel<<<dim3((nq + 7) / 8, b), 256, 0, s>>>(mine, m.q_pos, m.q_seg, m.q_pre, shape->lq, nq);
  plan_meta_kernel<<<dim3((nk + 7) / 8, b), 256, 0, s>>>(mine + (size_t)b * nq, m.kv_pos, m.kv_seg, m.kv_pre, shape->lk, nk);
  count_launch(2);
  if ((e = cudaGetLastError()) != cudaSuccess) return bail(fail_cuda(e, "plan_meta_kernel"));
  // the communicator's other traffic runs on the push stream: order the all-gather after it
  if ((e = cudaEventRecord(ring->ev_push_tail, ring->push_stream)) != cudaSuccess ||
      (e = cudaStreamWaitEvent(s, ring->ev_push_tail, 0)) != cudaSuccess)
    return bail(fail_cuda(e, "cudaStreamWaitEvent"));
  NcclApi* api = nccl_api();
  ncclResult_t nr = api->AllGather(mine, all, per_rank * sizeof(TileMeta), ncclChar, ring->comm, s);
  if (nr != ncclSuccess) return bail(fail_nccl(nr, "ncclAllGather(plan)"));
  if ((e = cudaMemsetAsync(need_dev, 0, sizeof(int) * N * N * 5, s)) != cudaSuccess) return bail(fail_cuda(e, "cudaMemsetAsync"));
  plan_need_kernel<<<N * N, 256, 0, s>>>(all, N, b, nq, nk, m.kinds, m.window, need_dev, need_dev + N * N);
  count_launch();
  if ((e = cudaGetLastError()) != cudaSuccess) return bail(fail_cuda(e, "plan_need_kernel"));
  if ((e = cudaMemcpyAsync(need_host.data(), need_dev, sizeof(int) * N * N * 5, cudaMemcpyDeviceToHost, s)) != cudaSuccess ||
      (e = cudaStreamSynchronize(s)) != cudaSuccess)
    return bail(fail_cuda(e, "plan readback"));
  // later NCCL traffic on the push stream comes after the all-gather
  if ((e = cudaEventRecord(ring->ev_start, s)) != cudaSuccess ||
      (e = cudaStreamWaitEvent(ring->push_stream, ring->ev_start, 0)) != cudaSuccess)
    return bail(fail_cuda(e, "cudaStreamWaitEvent"));
  for (size_t i = 0; i < (size_t)N * N; ++i) plan->need[i] = need_host[i] ? 1 : 0;
  for (int r = 0; r < N; ++r) plan->need[(size_t)r * N + r] = 1;  // the own block always runs
  plan->lk = shape->lk;
  plan->rows.assign(need_host.begin() + (size_t)N * N, need_host.end());
  cleanup();
  *out = plan;
  return 0;
}

void ra_ring_plan_destroy(ra_ring_plan_t* plan) { delete plan; }

int ra_ring_plan_need(const ra_ring_plan_t* plan, int32_t q_rank, int32_t kv_rank) {
  if (!plan) return fail(-6, "plan is NULL");
  if (q_rank < 0 || kv_rank < 0 || q_rank >= plan->nranks || kv_rank >= plan->nranks) return fail(-33, "bad rank");
  return plan->need[(size_t)q_rank * plan->nranks + kv_rank];
}

int ra_ring_plan_rows(const ra_ring_plan_t* plan, int32_t q_rank, int32_t kv_rank, int32_t runs[4]) {
  if (!plan || !runs) return fail(-6, "plan or result pointer is NULL");
  if (q_rank < 0 || kv_rank < 0 || q_rank >= plan->nranks || kv_rank >= plan->nranks) return fail(-33, "bad rank");
  const int chunks = (plan->lk + 127) / 128;
  if (plan->rows.empty()) {  // no mask to summarise: the whole block
    runs[0] = 0, runs[1] = plan->lk, runs[2] = runs[3] = 0;
    return 0;
  }
  for (int i = 0; i < 4; ++i) {
    const int v = plan->rows[((size_t)q_rank * plan->nranks + kv_rank) * 4 + i] * 128;
    runs[i] = v > plan->lk ? plan->lk : v;
  }
  (void)chunks;
  return 0;
}

int ra_ring_use_plan(ra_ring_t* ring, const ra_ring_plan_t* plan) {
  if (!ring) return fail(-30, "ring handle is NULL");
  if (plan && plan->nranks != ring->nranks) return fail(-39, "the plan was made for a ring of %d ranks", plan->nranks);
  ring->plan = plan;
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
  RA_NCCL(api->GroupStart(), "ncclGroupStart");
  for (int i = 0; i < n; ++i) {
    if (nbytes[i] <= 0) continue;
    RA_NCCL(api->Send(src[i], (size_t)nbytes[i], ncclChar, to, ring->comm, stream), "ncclSend");
    RA_NCCL(api->Recv(dst[i], (size_t)nbytes[i], ncclChar, from, ring->comm, stream), "ncclRecv");
  }
  RA_NCCL(api->GroupEnd(), "ncclGroupEnd");
  return 0;
}

}  // extern "C"
