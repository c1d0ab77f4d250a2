/*
 * ring_attention_b200 -- C ABI of the B200 (sm_100a) ring-attention engine.
 *
 * Every entry point is plain C: raw device pointers, sizes, strides and a CUDA stream
 * passed as void*.  No exceptions cross this boundary.  Return value: 0 = ok;
 * negative = argument error found on the host before anything was launched;
 * positive = CUDA / NCCL error code class (see RA_ERR_*).  ra_last_error_string()
 * gives the text for the calling thread's last failure.
 *
 * Tensors are addressed as [batch, length, heads, head_dim] with explicit element
 * strides for batch, length and heads; head_dim is contiguous.  That covers both the
 * reference's public layout "b l h d" (ring_attention/ring.py:80-82) and its internal
 * layout "b h l d" (ring.py:96-98) without a copy.
 *
 * Citations "ring.py:NN", "ring_kernel.py:NN" refer to files under ring_attention/ of
 * jondeaton/ring-attention-jax-pallas, the project this library is a drop-in for.
 */
#ifndef RING_ATTENTION_B200_H_
#define RING_ATTENTION_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RA_VERSION 1

/* element types of q, k, v, out, dout, dq, dk, dv */
#define RA_DTYPE_F32 0
#define RA_DTYPE_BF16 1

/* error classes (positive return values) */
#define RA_ERR_CUDA 1
#define RA_ERR_NCCL 2
#define RA_ERR_DEVICE_STATUS 3 /* a kernel reported a bounded wait that ran out */

/* score-mod kinds, OR-ed into ra_score_mod_t.kinds */
#define RA_MOD_CAUSAL 1u   /* keep kv_pos <= q_pos              (ring.py:394-397) */
#define RA_MOD_SEGMENT 2u  /* keep q_seg == kv_seg              (ring.py:388-391) */
#define RA_MOD_PREFIX 4u   /* keep (q_pre & kv_pre) | causal    (ring.py:399-406) */
#define RA_MOD_ALIBI 8u    /* add -slope[h] * (q_pos - kv_pos)  (a bias_fn, ring.py:107) */
#define RA_MOD_WINDOW 16u  /* keep q_pos - kv_pos < window      (a bias_fn, ring.py:107) */
#define RA_MOD_DENSE 32u   /* add a materialised bias tile      (ring.py:60-61) */
/* Gradients of a (batch, head) that has a query row which sees no key at all.  The reference
 * forms p = exp(s + bias - L) with s + bias = -inf and L = -inf for every pair of such a row
 * (ring.py:146): NaN, which reaches dQ of that row and, through the sums over queries, dK and dV
 * of EVERY key of that (batch, head), in every block of the ring.  The compiled-in masks define
 * p = 0 on a masked pair instead, so such rows contribute nothing (the useful behaviour:
 * padding rows do not destroy a batch).  With this bit set the backward calls reproduce the
 * reference: after each block, dQ of the rows whose L is -inf and dK, dV of the whole
 * (batch, head) are set to NaN.  It costs one more small kernel per block, switches off the
 * ring-of-one shortcut that writes dK/dV straight in the result type, and makes the ring calls
 * ignore a plan (the reference runs every step).  The dense-tile path (RA_MOD_DENSE) has the
 * reference behaviour with or without it. */
#define RA_MOD_STRICT_NAN 64u

/* kernel families; RA_IMPL_AUTO picks tcgen05 whenever the shape allows it */
#define RA_IMPL_AUTO 0
#define RA_IMPL_SIMT 1    /* fp32 CUDA-core kernels: any shape, fp32-exact */
#define RA_IMPL_TCGEN05 2 /* bf16 tensor-core kernels: fails if the shape does not fit */

typedef struct ra_tensor {
  void* ptr;        /* device pointer to element [0,0,0,0] */
  int64_t stride_b; /* element strides; head_dim stride is 1 */
  int64_t stride_l;
  int64_t stride_h;
} ra_tensor_t;

typedef struct ra_shape {
  int32_t b;   /* batch */
  int32_t h;   /* heads (q, k and v share it: ring.py:59, 92-93) */
  int32_t lq;  /* query rows in this block / shard */
  int32_t lk;  /* key/value rows in this block / shard */
  int32_t dk;  /* head dim of q and k */
  int32_t dv;  /* head dim of v and out */
  int32_t dtype;
  float sm_scale; /* ring.py:287-288 default is 1/sqrt(dk); the caller resolves it */
} ra_shape_t;

/*
 * Score modification: the compiled-in replacements for the reference's bias_fn
 * (ring.py:107, 185-188, 376-409).  Per-token arrays are int32 [b, lq] / [b, lk],
 * contiguous.  Any pointer whose kind bit is clear may be NULL.
 */
typedef struct ra_score_mod {
  uint32_t kinds;
  int32_t window;
  const int32_t* q_pos;
  const int32_t* kv_pos;
  const int32_t* q_seg;
  const int32_t* kv_seg;
  const uint8_t* q_prefix;
  const uint8_t* kv_prefix;
  const float* alibi_slopes; /* [h] */
  const float* bias;         /* dense fp32 tile, element (b,h,i,j) at b*sb + h*sh + i*sq + j */
  int64_t bias_stride_b;
  int64_t bias_stride_h; /* 0 broadcasts one tile over heads (ring.py:409) */
  int64_t bias_stride_q;
} ra_score_mod_t;

/* ---- diagnostics ------------------------------------------------------------------ */
int ra_version(void);
const char* ra_last_error_string(void);
/* Select the kernel family for later calls from this thread (RA_IMPL_*). */
int ra_set_impl(int impl);
/* Which family the last block call of this thread ran (RA_IMPL_SIMT / RA_IMPL_TCGEN05). */
int ra_last_impl(void);
/* Number of kernels this library has launched since load (all threads). */
int64_t ra_launch_count(void);

/* Synchronises the current device, then reads and clears its kernel status word.  Every
 * wait inside the tcgen05 kernels (on an mbarrier fed by TMA, by the tensor pipe or by
 * other warps) is bounded; a wait that runs out sets a bit, the kernel drains and returns,
 * and this call then returns RA_ERR_DEVICE_STATUS with the bits in *bits (else 0). */
int ra_device_status(uint32_t* bits);

/* ---- block level: the reference's plug point ---------------------------------------
 * ra_fwd_block replaces fwd_block / _fwd_block (ring_kernel.py:123-199, ring.py:58-76):
 * one online-softmax update of the carried state (o, m, l) with one K/V block.
 * o is fp32 [b,h,lq,dv] contiguous and un-normalised; m, l are fp32 [b,h,lq].
 * The state is updated in place.  first != 0 means "state is (0, -inf, 0)" and the
 * incoming buffers are not read (ring.py:124-126). mod may be NULL (no bias).
 */
int ra_fwd_block(const ra_shape_t* shape, const ra_tensor_t* q, const ra_tensor_t* k,
                 const ra_tensor_t* v, const ra_score_mod_t* mod, float* o, float* m, float* l,
                 int first, void* stream);

/* ra_fwd_block_static: the tensor-core forward block for hosts that must not allocate.
 * It has no counterpart in the reference.  ra_fwd_block takes a few kilobytes of device
 * scratch per call from the stream-ordered allocator (the per-tile mask summaries).  A
 * caller that runs inside an XLA / JAX FFI custom call, where XLA's allocator already owns
 * nearly all device memory, or a server that has given all free memory to its own arena,
 * cannot rely on that succeeding.  This entry point does the same work with the scratch
 * in a fixed 512 KiB array inside the library (held by every GPU that loads the library,
 * until the process ends) and calls no allocating routine.
 *   - Arguments and results are those of ra_fwd_block; the caller still owns q, k, v, the
 *     score-mod arrays and the carried state (o, m, l).
 *   - It serves only calls the tcgen05 forward takes (bf16, head dim 64 or 128, lq and lk
 *     multiples of 128, no dense bias); anything else is refused with a negative code.
 *   - Limit: shape->b * (lq/128 + lk/128) <= RA_STATIC_MAX_TILES, else -41 and nothing runs.
 *     Calls without a mask or ALiBi (mod NULL or kinds 0) read no summaries, never touch the
 *     array and have no such limit.
 *   - The first call on each device looks up the device addresses of the array and of the
 *     library's status word (with that device current); make that first call outside any
 *     stream capture.
 *   - All calls share the array, which keeps the previous call's contents.  Each call
 *     rewrites every entry it later reads, so nothing needs clearing, but calls that
 *     overlap on the GPU (two streams, two threads) race on it: serialise them.
 */
#define RA_STATIC_MAX_TILES 16384
int ra_fwd_block_static(const ra_shape_t* shape, const ra_tensor_t* q, const ra_tensor_t* k,
                        const ra_tensor_t* v, const ra_score_mod_t* mod, float* o, float* m,
                        float* l, int first, void* stream);

/* out = o / l, L = m + log(l): ring.py:134-135.  out has the element type shape->dtype. */
int ra_fwd_finalize(const ra_shape_t* shape, const float* o, const float* m, const float* l,
                    const ra_tensor_t* out, float* lse, void* stream);

/* delta = rowsum(out * dout) in fp32 [b,h,lq]: _precompute_delta, ring_kernel.py:387-409. */
int ra_bwd_delta(const ra_shape_t* shape, const ra_tensor_t* out, const ra_tensor_t* dout,
                 float* delta, void* stream);

/* ra_bwd_block replaces bwd_block / _bwd_block (ring_kernel.py:202-297, ring.py:140-157):
 * adds this block's contributions to fp32 accumulators dq [b,h,lq,dk], dk [b,h,lk,dk],
 * dv [b,h,lk,dv] (contiguous; the caller zeroes them first, ring.py:198-200).
 * lse and delta are fp32 [b,h,lq].
 */
int ra_bwd_block(const ra_shape_t* shape, const ra_tensor_t* q, const ra_tensor_t* k,
                 const ra_tensor_t* v, const ra_score_mod_t* mod, const float* lse,
                 const float* delta, const ra_tensor_t* dout, float* dq, float* dk, float* dv,
                 void* stream);

/* Convert a contiguous fp32 [b,h,len,d] accumulator to a strided tensor of `dtype`
 * (the "b h l d -> b l h d" + cast at ring.py:208-210). */
int ra_cast_from_f32(int32_t b, int32_t h, int32_t len, int32_t d, const float* src,
                     const ra_tensor_t* dst, int32_t dtype, void* stream);

/* ---- ring level -------------------------------------------------------------------
 * A ring handle binds one GPU (the current device) to its place in a ring of nranks
 * processes, one per GPU, and owns the K/V staging buffers, the fp32 carried state and
 * the gradient accumulators.  It replaces the mesh axis named by axis_name together
 * with lax.ppermute / lax.psum (ring.py:41-55, 101, 180).  nccl_id is the
 * NCCL unique id shared by all ranks (ra_ring_unique_id on rank 0, then broadcast by
 * the host program); it is ignored when nranks == 1.
 */
typedef struct ra_ring ra_ring_t;

#define RA_UNIQUE_ID_BYTES 128
int ra_ring_unique_id(uint8_t id[RA_UNIQUE_ID_BYTES]);
int ra_ring_create(int32_t rank, int32_t nranks, const uint8_t nccl_id[RA_UNIQUE_ID_BYTES],
                   ra_ring_t** ring);
int ra_ring_destroy(ra_ring_t* ring);
int ra_ring_rank(const ra_ring_t* ring);
int ra_ring_size(const ra_ring_t* ring);

/* Which transport the ring ended up with: 0 = ring of one (none), 1 = peer copies over CUDA
 * IPC mappings, 2 = NCCL send/recv.  Peer copies are the default; the ring falls back to NCCL
 * as a whole (every rank agrees) when RA_TRANSPORT=nccl is set or when some rank cannot export
 * or map a peer's buffers (no peer access between two of the GPUs, GPUs of different nodes). */
int ra_ring_transport(const ra_ring_t* ring);

/* Allocates, ahead of time, everything ra_ring_fwd (and, with backward != 0, ra_ring_bwd)
 * keeps in the handle for calls of this shape: the fp32 carried state (ring.py:124-126), the
 * gradient accumulators (ring.py:198-200), the staging slots that receive the other ranks'
 * K/V blocks (the operands of ring.py:120) and dK/dV contributions, and, with the peer-copy
 * transport, the exchange and mapping of their IPC handles.  This is the only place where the
 * ring calls cudaMalloc and synchronises the device: after it, ring calls of the same or a
 * smaller shape allocate nothing and never synchronise (a host that runs inside a framework's
 * custom call can reserve at set-up).  Without it the first call at each larger shape does the
 * same work itself.  Collective when nranks > 1: every rank calls it with the same shape.
 * Only which kv-side arrays of mod are non-NULL matters (they travel with K/V); mod may be NULL. */
int ra_ring_reserve(ra_ring_t* ring, const ra_shape_t* shape, const ra_score_mod_t* mod, int32_t backward);

/* Bound of one wait for a peer (a K/V block or a dK/dV contribution that has not arrived, a
 * buffer a peer has not released), in milliseconds of SM clock at 2 GHz.  Default: the
 * environment variable RA_RING_WAIT_MS when the ring is created, else 10000.  A wait that runs
 * out sets bit 16 of the device status word (ra_device_status) and the ring's abort word: from
 * then on the ring's kernels neither wait nor announce anything to the peers, whose own waits
 * run out in turn.  What the call computed after the wait is undefined (a block that never
 * arrived was read, or a buffer a late peer still read was overwritten), and the flag counters
 * of the ranks are out of step: destroy the ring on every rank and create a new one. */
int ra_ring_set_wait_ms(ra_ring_t* ring, int32_t ms);
/* 1 when a wait of this ring has run out (synchronous small copy from the device), else 0. */
int ra_ring_aborted(ra_ring_t* ring);
/* Diagnostic: enqueues the ring's bounded wait on a counter that nothing ever advances, so that
 * the time-out path can be exercised without a peer (set a short bound first).  The ring is
 * aborted afterwards, exactly as after a real time-out. */
int ra_ring_probe_wait(ra_ring_t* ring, void* stream);

/* Host-only schedule: which rank's K/V block this rank works on at step t
 * ((rank - t) mod nranks: ring.py:54 with the scan of ring.py:128-132). */
int ra_ring_source(int32_t rank, int32_t nranks, int32_t step);

/* Fused ring forward: _ring_attention_fwd (ring.py:79-137).  q,k,v are this rank's
 * shards; out gets this rank's rows in shape->dtype, lse gets L (fp32 [b,h,lq]).
 * K/V (and the kv-side arrays of mod) of the other ranks are fetched over NVLink on a
 * side stream into a ring of staging slots while earlier blocks are computed.
 * Every rank of the ring must make the same call with the same shape.
 */
int ra_ring_fwd(ra_ring_t* ring, const ra_shape_t* shape, const ra_tensor_t* q,
                const ra_tensor_t* k, const ra_tensor_t* v, const ra_score_mod_t* mod,
                const ra_tensor_t* out, float* lse, void* stream);

/* Fused ring backward: _ring_attention_bwd (ring.py:160-211).  Q, dO, L, delta and dQ
 * stay on their rank; K/V blocks are fetched as in the forward and each step's dK/dV
 * contribution is sent to the block's owner, which sums them in fp32. */
int ra_ring_bwd(ra_ring_t* ring, const ra_shape_t* shape, const ra_tensor_t* q,
                const ra_tensor_t* k, const ra_tensor_t* v, const ra_tensor_t* out,
                const float* lse, const ra_tensor_t* dout, const ra_score_mod_t* mod,
                const ra_tensor_t* dq, const ra_tensor_t* dk, const ra_tensor_t* dv,
                void* stream);

/* Ring steps that the mask empties.  With document masks or a sliding window most (query shard,
 * K/V block) pairs of a long ring have no visible pair: the reference still builds the bias tile
 * and runs the block for them (ring.py:104-132, 183-206); here the block kernels skip every tile
 * of such a pair, but its K/V block and dK/dV contribution would still cross NVLink.  A plan
 * records which pairs have a visible pair at all, from 128-token summaries of the positions,
 * segment ids and prefix masks that every rank contributes.
 *   ra_ring_plan_create  collective over the ring (every rank calls it with its own shard's
 *                        arrays and the same shape); all-gathers the summaries and SYNCHRONISES
 *                        the stream once.  Make it once per set of masks, not per layer.
 *   ra_ring_use_plan     later ra_ring_fwd / ra_ring_bwd calls on this handle leave out the
 *                        transfers and block launches of empty pairs (plan == NULL: all run).
 *                        Every rank must use the same plan, and the masks passed to those calls
 *                        must be the ones the plan was made from.  The handle does not own the plan.
 *   ra_ring_plan_need    1 when the queries of q_rank see something in the block of kv_rank. */
typedef struct ra_ring_plan ra_ring_plan_t;
int ra_ring_plan_create(ra_ring_t* ring, const ra_shape_t* shape, const ra_score_mod_t* mod, void* stream,
                        ra_ring_plan_t** plan);
void ra_ring_plan_destroy(ra_ring_plan_t* plan);
int ra_ring_plan_need(const ra_ring_plan_t* plan, int32_t q_rank, int32_t kv_rank);
/* The plan also bounds WHICH rows of a needed block matter: up to two runs of K/V rows (one in
 * each half of the block, in 128-row units) outside which the queries of q_rank see nothing.
 * Under a plan only those rows of K and V travel (the small per-token arrays always travel
 * whole) and only those rows of the dK/dV contribution come back and are summed: a sliding
 * window or a document boundary inside a block moves a halo, not the block (the reference
 * rotates whole blocks, ring.py:120, :195).  runs = {first0, end0, first1, end1} in rows;
 * an empty run has first >= end.  Row runs need k and v laid out [b, l, h, d]; other dense
 * layouts travel whole. */
int ra_ring_plan_rows(const ra_ring_plan_t* plan, int32_t q_rank, int32_t kv_rank, int32_t runs[4]);
int ra_ring_use_plan(ra_ring_t* ring, const ra_ring_plan_t* plan);

/* Rotate caller-owned buffers one place round the ring (rank i -> rank i+1), the
 * _rotate_block of ring.py:41-55, for the arbitrary-bias_fn path that loops on the host.
 * Sends nbytes from each src[i] and receives into dst[i]; n buffers per call. */
int ra_ring_rotate(ra_ring_t* ring, int32_t n, const void* const* src, void* const* dst,
                   const int64_t* nbytes, void* stream);

/* Milliseconds this rank's block kernels were held up by transfers during the last forward
 * (backward == 0) or backward (backward != 0) ring call of this handle: the time a compute lane
 * waited for a K/V block or for the final contribution sums while no block kernel of the rank
 * was running.  Also the total device time of that call.  Both need ra_ring_set_timing(ring, 1)
 * and synchronise on the call's end when read. */
int ra_ring_set_timing(ra_ring_t* ring, int32_t on);
int ra_ring_last_timing(ra_ring_t* ring, int32_t backward, float* total_ms, float* exposed_comm_ms);
/* Device time during which block kernels (ra_fwd_block / ra_bwd_block work) of the last
 * forward (backward == 0) or backward (backward != 0) ring call of this handle were running
 * (adjacent steps run on two streams and overlap: the union is taken), and how many launches
 * there were.  Timing must be on; the two directions are kept
 * apart so that a forward + backward step can be queried once, after it ended. */
int ra_ring_last_block_ms(ra_ring_t* ring, int32_t backward, float* block_ms, int32_t* launches);
/* The same call as a timeline: [begin, end] in ms from the call's start of every block launch
 * (in launch order; launches of the two compute lanes overlap) and of every wait for a transfer,
 * at most max_items of each (blocks and waits hold 2 * max_items floats).  Timing must be on. */
int ra_ring_last_timeline(ra_ring_t* ring, int32_t backward, int32_t max_items, float* blocks, int32_t* n_blocks,
                          float* waits, int32_t* n_waits);
/* Peer-copy transport: bytes this rank pushed to other ranks (K/V blocks, and dK/dV
 * contributions in the backward: the traffic of ring.py:120 and :195) during the last forward /
 * backward ring call, and the device time of those copies on the transfer stream, event to
 * event.  bytes / push_ms is the NVLink rate per direction the rotation achieved.  Timing
 * must be on. */
int ra_ring_last_push(ra_ring_t* ring, int32_t backward, double* bytes, float* push_ms);

#ifdef __cplusplus
}
#endif
#endif /* RING_ATTENTION_B200_H_ */
