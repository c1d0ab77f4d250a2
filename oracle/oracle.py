"""CPU oracle for ring attention: TEST INFRASTRUCTURE ONLY.

This file restates, in NumPy, the arithmetic of the reference project
(jondeaton/ring-attention-jax-pallas).  It exists so that the CUDA engine can be
checked against an independent statement of the same math, and so that a CPU
baseline can be timed.  Nothing in the product path may import it: only the test
suite, the smoke check and the benchmark's cpu-baseline / reference arm do.

Pinning.  The reference stores no golden arrays; its tests draw inputs from
`jax.random` and assert one property: ring attention equals dense softmax attention
and its gradients (ring_attention/ring_test.py:26-42, :97-98, :165-171, :273-274,
:298-300, :378).  JAX is not installable here, so the JAX/Pallas program itself cannot
be run.  What pins this oracle:
(1) the reference's own ring.py and ring_kernel.py, imported unmodified and run on a
    NumPy stand-in for the JAX and Pallas names they use (tests/golden/jax_on_numpy.py;
    8 virtual devices): tests/test_reference_run.py holds this oracle to their out, L,
    dQ, dK, dV, NaN and inf patterns included, at 1e-11 for `block_impl="jax"` in
    float64 and to float32 rounding for the Pallas kernels, and tests/golden/*.npz are
    outputs of that run (tests/test_oracle.py::test_golden_fixtures);
(2) the ring emulation below equals the dense restatement of the reference test's
    `mha` at every shape the reference tests use, to 1e-12 in float64;
(3) the dense restatement equals torch's CPU scaled_dot_product_attention and torch
    autograd gradients, an independent implementation.
Not pinned: XLA's / Triton's own float32 rounding and Pallas' real runtime (in that
byte-for-byte sense: "parity unpinned").

Each function cites the reference lines it follows.
"""

from __future__ import annotations

import math
from typing import Callable, Optional

import numpy as np

NEG_INF = -np.inf


# --------------------------------------------------------------------------------------
# Dense attention: ring_attention/ring_test.py:26-42 (`mha`), layout [b, l, h, d].
# --------------------------------------------------------------------------------------
def mha(q, k, v, bias=None, sm_scale=None, dtype=np.float64, return_lse=False):
    """softmax(q k^T * scale + bias) v.  ring_test.py:26-42 uses scale 1/sqrt(dk)."""
    q = np.asarray(q, dtype)
    k = np.asarray(k, dtype)
    v = np.asarray(v, dtype)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    z = np.einsum("bihd,bjhd->bhij", q, k) * dtype(sm_scale)
    if bias is not None:
        z = z + np.asarray(bias, dtype)
    with np.errstate(invalid="ignore", divide="ignore"):
        m = np.max(z, axis=-1, keepdims=True)
        p = np.exp(z - m)  # rows that are all -inf give exp(nan) = nan, like jax.nn.softmax
        l = np.sum(p, axis=-1, keepdims=True)
        a = p / l
        out = np.einsum("bhij,bjhd->bihd", a, v)
        if return_lse:
            # a row that sees no key: the ring carries m = -inf, l = 0 and ends with
            # L = -inf + log 0 = -inf (ring.py:66-69, 135), while out = 0 / 0 = NaN
            lse = np.where(np.isneginf(m), -np.inf, m + np.log(l))[..., 0]
            return out, lse
    return out


def mha_grads(q, k, v, do, bias=None, sm_scale=None, dtype=np.float64):
    """Gradients of sum(do * mha(q,k,v)) wrt q,k,v (the loss of ring_test.py:136,160)."""
    q = np.asarray(q, dtype)
    k = np.asarray(k, dtype)
    v = np.asarray(v, dtype)
    do = np.asarray(do, dtype)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    z = np.einsum("bihd,bjhd->bhij", q, k) * dtype(sm_scale)
    if bias is not None:
        z = z + np.asarray(bias, dtype)
    with np.errstate(invalid="ignore", divide="ignore"):
        m = np.max(z, axis=-1, keepdims=True)
        p = np.exp(z - m)
        a = p / np.sum(p, axis=-1, keepdims=True)
        out = np.einsum("bhij,bjhd->bihd", a, v)
        dv = np.einsum("bhij,bihd->bjhd", a, do)
        dp = np.einsum("bihd,bjhd->bhij", do, v)
        delta = np.einsum("bihd,bihd->bhi", do, out)[..., None]
        ds = a * (dp - delta) * dtype(sm_scale)
        dq = np.einsum("bhij,bjhd->bihd", ds, k)
        dk = np.einsum("bhij,bihd->bjhd", ds, q)
    return dq, dk, dv


# --------------------------------------------------------------------------------------
# Block math, layout [b, h, l, d]: ring_attention/ring.py:58-76 and :140-157.
# --------------------------------------------------------------------------------------
def fwd_block(q, k, v, bias, o, m_prev, l, sm_scale):
    """One online-softmax block update.  Follows ring.py:58-76 line by line."""
    s = np.einsum("bhqd,bhkd->bhqk", q, k) * sm_scale  # ring.py:59
    if bias is not None:
        s = s + bias  # ring.py:60-61
    with np.errstate(invalid="ignore"):
        m = np.maximum(m_prev, np.max(s, axis=-1))  # ring.py:63
        correction = np.exp(m_prev - m)  # ring.py:65
        correction = np.where(np.isneginf(m) & np.isneginf(m_prev), 0, correction)  # :66
        p = np.exp(s - m[..., None])  # ring.py:68
        p = np.where(np.isneginf(m)[..., None], 0, p)  # ring.py:69
    pv = np.einsum("bhqk,bhkd->bhqd", p, v)  # ring.py:70
    o = o * correction[..., None] + pv  # ring.py:72
    l = correction * l + np.sum(p, axis=-1)  # ring.py:75
    return o, m, l


def bwd_block(q, k, v, bias, o, L, do, sm_scale):
    """Block VJP.  Follows ring.py:140-157."""
    s = np.einsum("bhqd,bhkd->bhqk", q, k) * sm_scale  # ring.py:142
    if bias is not None:
        s = s + bias
    with np.errstate(invalid="ignore"):
        p = np.exp(s - L[..., None])  # ring.py:146
        dv = np.einsum("bhqk,bhqd->bhkd", p, do)  # ring.py:148
        dp = np.einsum("bhqd,bhkd->bhqk", do, v)  # ring.py:150
        delta = np.sum(do * o, axis=-1, keepdims=True)  # ring.py:151
        ds = p * (dp - delta) * sm_scale  # ring.py:152
        dq = np.einsum("bhqk,bhkd->bhqd", ds, k)  # ring.py:154
        dk = np.einsum("bhqk,bhqd->bhkd", ds, q)  # ring.py:155
    return dq, dk, dv


def finalize(o, m, l):
    """out = o / l ; L = m + log l.  ring.py:134-135."""
    with np.errstate(invalid="ignore", divide="ignore"):
        return o / l[..., None], m + np.log(l)


# --------------------------------------------------------------------------------------
# Ring schedule over N virtual ranks: ring.py:79-137 (forward), :160-211 (backward),
# rotation ring.py:41-55 (rank i sends to rank (i+1) % N).
# --------------------------------------------------------------------------------------
def _rotate(blocks):
    """Cyclic +1 shift over the rank axis: what rank i held is now on rank i+1 (ring.py:51-55)."""
    return [blocks[(r - 1) % len(blocks)] for r in range(len(blocks))]


def _bhld(x):
    return np.ascontiguousarray(np.transpose(x, (0, 2, 1, 3)))


def ring_attention_fwd(
    q_shards,
    k_shards,
    v_shards,
    bias_fn: Optional[Callable] = None,
    q_kwargs=None,
    kv_kwargs=None,
    sm_scale=None,
    dtype=np.float64,
    block_fn=fwd_block,
):
    """Forward over N = len(q_shards) virtual ranks; shards are [b, c, h, d] (ring.py:80-82).

    q_kwargs / kv_kwargs: per-rank lists of dicts of per-token arrays [b, c] that travel
    with the queries / keys (ring.py:107,120).  Returns per-rank (out [b,c,h,dv], L [b,h,c]).
    """
    n = len(q_shards)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q_shards[0].shape[-1])  # ring.py:287-288
    q_kwargs = q_kwargs or [{} for _ in range(n)]
    kv_kwargs = kv_kwargs or [{} for _ in range(n)]
    q = [_bhld(np.asarray(x, dtype)) for x in q_shards]  # ring.py:96-98
    k = [_bhld(np.asarray(x, dtype)) for x in k_shards]
    v = [_bhld(np.asarray(x, dtype)) for x in v_shards]
    kvk = list(kv_kwargs)
    o = [np.zeros(q[r].shape[:3] + (v[r].shape[-1],), dtype) for r in range(n)]  # ring.py:124
    l = [np.zeros(q[r].shape[:3], dtype) for r in range(n)]  # ring.py:125
    m = [np.full(q[r].shape[:3], NEG_INF, dtype) for r in range(n)]  # ring.py:126
    for _ in range(n):  # ring.py:128-132
        for r in range(n):
            bias = bias_fn(**q_kwargs[r], **kvk[r]) if bias_fn is not None else None
            o[r], m[r], l[r] = block_fn(q[r], k[r], v[r], bias, o[r], m[r], l[r], sm_scale)
        k, v, kvk = _rotate(k), _rotate(v), _rotate(kvk)  # ring.py:120
    outs, lses = [], []
    for r in range(n):
        out, L = finalize(o[r], m[r], l[r])
        outs.append(np.transpose(out, (0, 2, 1, 3)))  # ring.py:137
        lses.append(L)
    return outs, lses


def ring_attention_bwd(
    q_shards,
    k_shards,
    v_shards,
    out_shards,
    lse_shards,
    do_shards,
    bias_fn=None,
    q_kwargs=None,
    kv_kwargs=None,
    sm_scale=None,
    dtype=np.float64,
    block_fn=bwd_block,
):
    """Backward over N virtual ranks: K,V,dK,dV stay, the query bundle travels (ring.py:183-206)."""
    n = len(q_shards)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q_shards[0].shape[-1])
    q_kwargs = q_kwargs or [{} for _ in range(n)]
    kv_kwargs = kv_kwargs or [{} for _ in range(n)]
    q = [_bhld(np.asarray(x, dtype)) for x in q_shards]
    k = [_bhld(np.asarray(x, dtype)) for x in k_shards]
    v = [_bhld(np.asarray(x, dtype)) for x in v_shards]
    o = [_bhld(np.asarray(x, dtype)) for x in out_shards]
    do = [_bhld(np.asarray(x, dtype)) for x in do_shards]  # ring.py:173
    L = [np.asarray(x, dtype) for x in lse_shards]
    qk = list(q_kwargs)
    dq = [np.zeros_like(x) for x in q]  # ring.py:198-200
    dk = [np.zeros_like(x) for x in k]
    dv = [np.zeros_like(x) for x in v]
    for _ in range(n):  # ring.py:202-206
        for r in range(n):
            bias = bias_fn(**qk[r], **kv_kwargs[r]) if bias_fn is not None else None
            dq_, dk_, dv_ = block_fn(q[r], k[r], v[r], bias, o[r], L[r], do[r], sm_scale)
            dq[r] = dq[r] + dq_  # ring.py:191-193
            dk[r] = dk[r] + dk_
            dv[r] = dv[r] + dv_
        q, o, dq, do, L, qk = (_rotate(x) for x in (q, o, dq, do, L, qk))  # ring.py:195
    t = lambda xs: [np.transpose(x, (0, 2, 1, 3)) for x in xs]  # ring.py:208-210
    return t(dq), t(dk), t(dv)


# --------------------------------------------------------------------------------------
# Bias builders.
# --------------------------------------------------------------------------------------
def self_attention_bias(
    causal: bool,
    q_segment_ids=None,
    kv_segment_ids=None,
    q_positions=None,
    kv_positions=None,
    q_prefix_mask=None,
    kv_prefix_mask=None,
):
    """The block bias of ring_self_attention: ring.py:376-409.  Returns [b, 1, lq, lk]."""
    mask = np.array(True)
    if q_segment_ids is not None:
        mask = mask & (q_segment_ids[:, :, None] == kv_segment_ids[:, None, :])  # ring.py:390-391
    if causal:
        mask = mask & (kv_positions[:, None, :] <= q_positions[:, :, None])  # ring.py:396-397
    elif q_prefix_mask is not None:
        pre = q_prefix_mask[:, :, None].astype(bool) & kv_prefix_mask[:, None, :].astype(bool)
        cau = kv_positions[:, None, :] <= q_positions[:, :, None]
        mask = mask & (pre | cau)  # ring.py:404-406
    bias = np.where(mask, 0.0, NEG_INF)  # ring.py:408
    return bias[:, None, :, :]  # ring.py:409


def score_mod_bias(
    b,
    h,
    q_positions=None,
    kv_positions=None,
    q_segment_ids=None,
    kv_segment_ids=None,
    q_prefix_mask=None,
    kv_prefix_mask=None,
    causal=False,
    alibi_slopes=None,
    window=0,
):
    """Dense [b, h, lq, lk] bias for the engine's compiled-in score-mod variants.

    causal / segment / prefix follow ring.py:386-408.  ALiBi adds
    -slope[h] * (q_pos - kv_pos); a sliding window of W keeps pairs with
    q_pos - kv_pos < W (combined with causal this is 0 <= q_pos - kv_pos < W).
    These two have no counterpart in the reference other than through a user bias_fn
    (ring.py:107); they are defined here as that bias_fn would compute them.
    """
    lq = (q_positions if q_positions is not None else q_segment_ids).shape[1]
    lk = (kv_positions if kv_positions is not None else kv_segment_ids).shape[1]
    mask = np.ones((b, 1, lq, lk), bool)
    if q_segment_ids is not None:
        mask &= (q_segment_ids[:, :, None] == kv_segment_ids[:, None, :])[:, None]
    rel = None
    if q_positions is not None:
        rel = (q_positions[:, :, None].astype(np.int64) - kv_positions[:, None, :].astype(np.int64))[:, None]
    if causal:
        mask &= rel >= 0
    elif q_prefix_mask is not None:
        pre = (q_prefix_mask[:, :, None].astype(bool) & kv_prefix_mask[:, None, :].astype(bool))[:, None]
        mask &= pre | (rel >= 0)
    if window:
        mask &= rel < window
    bias = np.zeros((b, h, lq, lk), np.float64)
    if alibi_slopes is not None:
        bias = bias - np.asarray(alibi_slopes, np.float64)[None, :, None, None] * rel
    return np.where(mask, bias, NEG_INF)


def alibi_slopes(h, zero_based=False):
    """Slopes 2^(-8(i+1)/h) for head i (the usual ALiBi convention); zero_based gives 2^(-8i/h)."""
    i = np.arange(h, dtype=np.float64)
    return 2.0 ** (-8.0 * (i if zero_based else i + 1) / h)


def pack_documents(total_len, lo, hi, seed):
    """Segment ids [total_len] from document lengths drawn uniformly in [lo, hi] until full."""
    rng = np.random.default_rng(seed)
    ids = np.empty(total_len, np.int32)
    pos, doc = 0, 0
    lens = []
    while pos < total_len:
        n = int(rng.integers(lo, hi + 1))
        n = min(n, total_len - pos)
        ids[pos : pos + n] = doc
        lens.append(n)
        pos += n
        doc += 1
    return ids, np.asarray(lens, np.int64)


# --------------------------------------------------------------------------------------
# Exact pair counters for FLOP accounting (pairs * 4d fwd, * 10d bwd).
# --------------------------------------------------------------------------------------
def pairs_causal(s):
    return s * (s + 1) // 2


def pairs_documents(lens):
    lens = np.asarray(lens, np.int64)
    return int(np.sum(lens * (lens + 1) // 2))


def pairs_window(s, w):
    i = np.arange(s, dtype=np.int64)
    return int(np.sum(np.minimum(i + 1, w)))


def pairs_from_bias(bias):
    return int(np.sum(~np.isneginf(bias)))


# --------------------------------------------------------------------------------------
# Convenience: split a global [b, S, ...] array into N contiguous shards on axis 1.
# --------------------------------------------------------------------------------------
def shard(x, n):
    return [np.ascontiguousarray(s) for s in np.split(np.asarray(x), n, axis=1)]


def unshard(xs, axis=1):
    return np.concatenate(xs, axis=axis)


# --------------------------------------------------------------------------------------
# BLAS-backed restatement of the same block math, for the TIMED CPU baseline only.
# np.einsum above does not call a threaded GEMM; np.matmul does, so this is the form that
# uses all host cores.  tests/test_oracle.py checks it against fwd_block / bwd_block.
# --------------------------------------------------------------------------------------
def fwd_block_mm(q, k, v, bias, o, m_prev, l, sm_scale):
    """ring.py:58-76 with batched GEMMs."""
    s = np.matmul(q, np.swapaxes(k, -1, -2)) * q.dtype.type(sm_scale)
    if bias is not None:
        s += bias
    with np.errstate(invalid="ignore"):
        m = np.maximum(m_prev, np.max(s, axis=-1))
        correction = np.exp(m_prev - m)
        correction = np.where(np.isneginf(m) & np.isneginf(m_prev), 0, correction).astype(q.dtype)
        np.subtract(s, m[..., None], out=s)
        np.exp(s, out=s)
        p = np.where(np.isneginf(m)[..., None], 0, s).astype(q.dtype)
    o = o * correction[..., None] + np.matmul(p, v)
    l = correction * l + np.sum(p, axis=-1)
    return o, m, l


def bwd_block_mm(q, k, v, bias, o, L, do, sm_scale):
    """ring.py:140-157 with batched GEMMs."""
    s = np.matmul(q, np.swapaxes(k, -1, -2)) * q.dtype.type(sm_scale)
    if bias is not None:
        s += bias
    with np.errstate(invalid="ignore"):
        p = np.exp(s - L[..., None])
        dv = np.matmul(np.swapaxes(p, -1, -2), do)
        dp = np.matmul(do, np.swapaxes(v, -1, -2))
        delta = np.sum(do * o, keepdims=True, axis=-1)
        ds = p * (dp - delta) * q.dtype.type(sm_scale)
        dq = np.matmul(ds, k)
        dk = np.matmul(np.swapaxes(ds, -1, -2), q)
    return dq, dk, dv


def causal_flops(b, h, s, d, fwd=True, bwd=True):
    """Algorithmic FLOPs of causal attention: 4d per visible pair forward, 10d backward."""
    per_pair = (4 * d if fwd else 0) + (10 * d if bwd else 0)
    return b * h * pairs_causal(s) * per_pair


def timed_cpu_ring_causal(b, h, s, d, nranks, seed=0, dtype=np.float32):
    """One forward+backward of causal ring attention over `nranks` virtual ranks on the
    host (the reference's algorithm, ring.py:79-211, BLAS block math).  Returns seconds."""
    import time

    rng = np.random.default_rng(seed)
    mk = lambda: rng.standard_normal((b, s, h, d)).astype(dtype)
    q, k, v, do = mk(), mk(), mk(), mk()
    pos = np.broadcast_to(np.arange(s, dtype=np.int32), (b, s))
    fn = lambda **kw: self_attention_bias(True, **kw).astype(dtype)
    qk = [{"q_positions": p} for p in shard(pos, nranks)]
    kk = [{"kv_positions": p} for p in shard(pos, nranks)]
    qs, ks, vs, dos = (shard(x, nranks) for x in (q, k, v, do))
    t0 = time.perf_counter()
    outs, lses = ring_attention_fwd(qs, ks, vs, fn, qk, kk, dtype=dtype, block_fn=fwd_block_mm)
    ring_attention_bwd(qs, ks, vs, outs, lses, dos, fn, qk, kk, dtype=dtype, block_fn=bwd_block_mm)
    return time.perf_counter() - t0


# --------------------------------------------------------------------------------------
# Sampled rows of a long sequence.  A dense float64 oracle over 32k - 1M tokens is out of
# reach, but single rows are cheap: a query row attends to all keys in O(S d), and the
# gradient of a key row needs L and delta only of the queries that see it.  Same math as
# mha / mha_grads above (ring_test.py:26-42 and its jax.grad), one (batch, head) at a time,
# tokens in position order (token i has position i), with the masks of score_mod_bias.
# --------------------------------------------------------------------------------------
def _visible(qi, kj, seg, window, causal):
    """[len(qi), len(kj)] mask of visible pairs between query positions qi and key positions kj."""
    rel = qi[:, None] - kj[None, :]
    vis = np.ones(rel.shape, bool)
    if causal:
        vis &= rel >= 0
    if seg is not None:
        vis &= seg[qi][:, None] == seg[kj][None, :]
    if window:
        vis &= rel < window
    return vis, rel


def sampled_rows(q, k, v, do, scale, q_rows, k_rows, seg=None, window=0, slope=None, causal=True, blk=1024,
                 score_dtype=np.float64):
    """q, k, v, do: [S, d] float64 of one (batch, head), token i at position i.

    Returns out, L, dq of the query rows `q_rows` and dk, dv of the key rows `k_rows`
    (either list may be empty).  `slope`: ALiBi slope of this head (bias -slope * (i - j)).
    `score_dtype` float32 makes the wide score products of the dk/dv part cheaper; the
    per-row parts are always float64.
    """
    S = q.shape[0]
    q_rows = np.asarray(q_rows, np.int64)
    k_rows = np.asarray(k_rows, np.int64)
    allk = np.arange(S)
    res = {}

    def scores(qi, lo, hi, dtype=np.float64):
        kj = allk[lo:hi]
        s = (q[qi].astype(dtype) @ k[lo:hi].astype(dtype).T).astype(np.float64) * scale
        vis, rel = _visible(qi, kj, seg, window, causal)
        if slope is not None:
            s = s - slope * rel
        return np.where(vis, s, NEG_INF), vis

    seg_sorted = seg is not None and bool(np.all(np.diff(seg) >= 0))  # packed documents

    def key_range(qi):
        """A range of keys that holds every key some query of qi can see (only a cost bound)."""
        lo, hi = 0, S
        if causal:
            hi = int(qi.max()) + 1
        if window and causal:
            lo = max(0, int(qi.min()) - window + 1)
        if seg_sorted:
            lo = max(lo, int(np.searchsorted(seg, seg[qi.min()], side="left")))
            hi = min(hi, int(np.searchsorted(seg, seg[qi.max()], side="right")))
        return lo, hi

    if q_rows.size:
        outs, Ls, dqs = [], [], []
        for i in q_rows:
            qi = np.array([i])
            lo, hi = key_range(qi)
            s, _ = scores(qi, lo, hi)
            s = s[0]
            with np.errstate(invalid="ignore", divide="ignore"):
                m = s.max()
                p = np.exp(s - m)
                l = p.sum()
                a = p / l
                o = a @ v[lo:hi]
                dp = v[lo:hi] @ do[i]
                ds = a * (dp - do[i] @ o) * scale
                outs.append(o)
                Ls.append(m + np.log(l))
                dqs.append(ds @ k[lo:hi])
        res["out"], res["L"], res["dq"] = np.array(outs), np.array(Ls), np.array(dqs)

    if k_rows.size:
        # queries that see at least one sampled key
        seen = np.zeros(S, bool)
        for j in k_rows:
            vis, _ = _visible(allk, np.array([j]), seg, window, causal)
            seen |= vis[:, 0]
        I = np.nonzero(seen)[0]
        L = np.full(S, np.nan)
        delta = np.full(S, np.nan)
        for c0 in range(0, I.size, blk):
            qi = I[c0:c0 + blk]
            lo, hi = key_range(qi)
            s, _ = scores(qi, lo, hi, score_dtype)
            m = s.max(-1)
            p = np.exp(s - m[:, None])
            l = p.sum(-1)
            L[qi] = m + np.log(l)
            delta[qi] = np.einsum("id,id->i", (p / l[:, None]) @ v[lo:hi], do[qi])
        dks, dvs = [], []
        for j in k_rows:
            vis, rel = _visible(I, np.array([j]), seg, window, causal)
            vis, rel = vis[:, 0], rel[:, 0]
            qi = I[vis]
            s = (q[qi] @ k[j]) * scale
            if slope is not None:
                s = s - slope * rel[vis]
            p = np.exp(s - L[qi])
            dvs.append(p @ do[qi])
            ds = p * (do[qi] @ v[j] - delta[qi]) * scale
            dks.append(ds @ q[qi])
        res["dk"], res["dv"] = np.array(dks), np.array(dvs)
    return res


def bf16_excess(got, want, atol=2e-2, rtol=1e-2):
    """Largest amount by which |got - want| exceeds atol + rtol * |want| (<= 0 means inside the bound)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float((np.abs(got - want) - (atol + rtol * np.abs(want))).max()) if want.size else float("-inf")
