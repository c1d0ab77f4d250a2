"""CPU tests that pin the oracle (oracle/oracle.py).

The reference's own tests hold no stored vectors; what they assert is that ring attention
equals dense softmax attention and its gradients at a fixed list of shapes
(ring_attention/ring_test.py:45-378).  Those assertions are replayed here on the oracle's
ring emulation, at the reference's shapes and with 8 virtual ranks, and the dense
restatement is checked against torch's CPU attention and autograd.
"""
import math

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.golden import make_golden as G

FWD_SHAPES = [(0, 24, 16, 1, 2), (1, 128, 64, 4, 64), (2, 64, 512, 4, 16), (3, 2048, 2048, 4, 128)]
BWD_SHAPES = FWD_SHAPES[:3] + [(3, 128, 2048, 2, 128), (3, 2048, 128, 2, 128)]


def _rand(seed, lq, lk, h, d, b=2):
    rng = np.random.default_rng(seed)
    mk = lambda l: rng.standard_normal((b, l, h, d))
    return mk(lq), mk(lk), mk(lk), mk(lq), rng


@pytest.mark.parametrize("seed,lq,lk,h,d", FWD_SHAPES)
def test_ring_forward_equals_dense(seed, lq, lk, h, d):
    """ring_test.py:45-98 on the oracle, float64."""
    if lq * lk > 1 << 21:
        lq, lk = lq // 4, lk // 4  # keep the CPU suite short; 8 ranks of 64 rows
    q, k, v, _, _ = _rand(seed, lq, lk, h, d)
    outs, lses = O.ring_attention_fwd(O.shard(q, 8), O.shard(k, 8), O.shard(v, 8))
    ref, ref_lse = O.mha(q, k, v, return_lse=True)
    np.testing.assert_allclose(O.unshard(outs), ref, rtol=0, atol=1e-12)
    np.testing.assert_allclose(O.unshard(lses, axis=2), ref_lse, rtol=0, atol=1e-12)


@pytest.mark.parametrize("seed,lq,lk,h,d", BWD_SHAPES)
def test_ring_backward_equals_dense(seed, lq, lk, h, d):
    """ring_test.py:101-171 on the oracle."""
    if lq * lk > 1 << 19:
        lq, lk = max(lq // 4, 32), max(lk // 4, 32)
    q, k, v, do, _ = _rand(seed, lq, lk, h, d)
    qs, ks, vs, dos = (O.shard(x, 8) for x in (q, k, v, do))
    outs, lses = O.ring_attention_fwd(qs, ks, vs)
    dq, dk, dv = O.ring_attention_bwd(qs, ks, vs, outs, lses, dos)
    rq, rk, rv = O.mha_grads(q, k, v, do)
    for a, r in ((dq, rq), (dk, rk), (dv, rv)):
        np.testing.assert_allclose(O.unshard(a), r, rtol=0, atol=1e-11)


@pytest.mark.parametrize("seed,lq,lk,h,d", FWD_SHAPES[:3])
def test_ring_bias_nan_pattern_and_grads(seed, lq, lk, h, d):
    """ring_test.py:174-300: independent random segment ids, user bias_fn, NaN pattern."""
    q, k, v, do, rng = _rand(seed, lq, lk, h, d)
    qseg = rng.integers(0, max(lq // 5, 1), (2, lq))
    kseg = rng.integers(0, max(lq // 5, 1), (2, lk))

    def bias_fn(q_segment_ids, kv_segment_ids):
        mask = q_segment_ids[:, :, None] == kv_segment_ids[:, None, :]
        return np.repeat(np.where(mask, 0.0, -np.inf)[:, None], h, axis=1)

    bias = bias_fn(qseg, kseg)
    ref = O.mha(q, k, v, bias)
    qs, ks, vs, dos = (O.shard(x, 8) for x in (q, k, v, do))
    qk = [{"q_segment_ids": s} for s in O.shard(qseg, 8)]
    kk = [{"kv_segment_ids": s} for s in O.shard(kseg, 8)]
    outs, lses = O.ring_attention_fwd(qs, ks, vs, bias_fn, qk, kk)
    out = O.unshard(outs)
    np.testing.assert_array_equal(np.isnan(out), np.isnan(ref))  # ring_test.py:273
    np.testing.assert_allclose(out, ref, rtol=0, atol=1e-12)
    dq, dk, dv = O.ring_attention_bwd(qs, ks, vs, outs, lses, dos, bias_fn, qk, kk)
    rq, rk, rv = O.mha_grads(q, k, v, do, bias)
    for a, r in ((dq, rq), (dk, rk), (dv, rv)):
        a = O.unshard(a)
        np.testing.assert_array_equal(np.isnan(a), np.isnan(r))
        np.testing.assert_allclose(a, r, rtol=0, atol=1e-11)


@pytest.mark.parametrize("seed,length,h,d", [(0, 16, 1, 2), (1, 128, 4, 64), (2, 512, 4, 16)])
def test_ring_self_attention_mask(seed, length, h, d):
    """ring_test.py:320-378: causal + random segment ids through the built-in mask."""
    q, k, v, _, rng = _rand(seed, length, length, h, d)
    seg = rng.integers(0, 5, (2, length))
    pos = np.broadcast_to(np.arange(length), (2, length))
    i = np.arange(length)
    mask = (seg[:, :, None] == seg[:, None, :]) & (i[None, :] <= i[:, None])  # ring_test.py:303-317
    ref = O.mha(q, k, v, np.where(mask, 0.0, -np.inf)[:, None])
    fn = lambda **kw: O.self_attention_bias(True, **kw)
    qk = [{"q_segment_ids": s, "q_positions": p} for s, p in zip(O.shard(seg, 8), O.shard(pos, 8))]
    kk = [{"kv_segment_ids": s, "kv_positions": p} for s, p in zip(O.shard(seg, 8), O.shard(pos, 8))]
    outs, _ = O.ring_attention_fwd(O.shard(q, 8), O.shard(k, 8), O.shard(v, 8), fn, qk, kk)
    np.testing.assert_allclose(O.unshard(outs), ref, rtol=0, atol=1e-12)


def test_prefix_mask_matches_brute_force():
    """ring.py:399-406 against a per-pair loop."""
    rng = np.random.default_rng(5)
    b, l = 2, 24
    seg = rng.integers(0, 2, (b, l))
    pos = np.broadcast_to(np.arange(l), (b, l))
    pre = rng.integers(0, 2, (b, l)).astype(bool)
    bias = O.self_attention_bias(False, seg, seg, pos, pos, pre, pre)
    for bb in range(b):
        for i in range(l):
            for j in range(l):
                vis = seg[bb, i] == seg[bb, j] and ((pre[bb, i] and pre[bb, j]) or j <= i)
                assert (bias[bb, 0, i, j] == 0) == vis
    dense = O.score_mod_bias(b, 3, pos, pos, seg, seg, pre, pre)
    np.testing.assert_array_equal(dense[:, 0], bias[:, 0])


def test_dense_matches_torch_sdpa_and_autograd():
    """The dense restatement against an independent implementation."""
    q, k, v, do, rng = _rand(11, 40, 56, 3, 16)
    bias = rng.standard_normal((2, 3, 40, 56))
    tq, tk, tv = (torch.tensor(x, requires_grad=True) for x in (q, k, v))
    out = torch.nn.functional.scaled_dot_product_attention(
        tq.transpose(1, 2), tk.transpose(1, 2), tv.transpose(1, 2), attn_mask=torch.tensor(bias)
    ).transpose(1, 2)
    (out * torch.tensor(do)).sum().backward()
    np.testing.assert_allclose(O.mha(q, k, v, bias), out.detach().numpy(), atol=1e-12)
    dq, dk, dv = O.mha_grads(q, k, v, do, bias)
    np.testing.assert_allclose(dq, tq.grad.numpy(), atol=1e-12)
    np.testing.assert_allclose(dk, tk.grad.numpy(), atol=1e-12)
    np.testing.assert_allclose(dv, tv.grad.numpy(), atol=1e-12)


def test_alibi_window_bias_and_pair_counts():
    b, h, s, w = 1, 4, 64, 9
    pos = np.arange(s)[None]
    slopes = O.alibi_slopes(h)
    bias = O.score_mod_bias(b, h, pos, pos, causal=True, alibi_slopes=slopes, window=w)
    for i in range(s):
        for j in range(s):
            vis = 0 <= i - j < w
            assert np.isneginf(bias[0, 1, i, j]) != vis
            if vis:
                assert bias[0, 1, i, j] == -slopes[1] * (i - j)
    assert O.pairs_from_bias(bias[:, :1]) == O.pairs_window(s, w)
    assert O.pairs_from_bias(O.score_mod_bias(b, 1, pos, pos, causal=True)) == O.pairs_causal(s)
    ids, lens = O.pack_documents(300, 10, 50, seed=3)
    assert lens.sum() == 300 and ids[-1] == len(lens) - 1
    docb = O.score_mod_bias(1, 1, np.arange(300)[None], np.arange(300)[None], ids[None], ids[None], causal=True)
    assert O.pairs_from_bias(docb) == O.pairs_documents(lens)


@pytest.mark.parametrize("name", list(G.CASES))
def test_golden_fixtures(name):
    """The committed fixtures are outputs of the reference's own code (run on the NumPy stand-in,
    see make_golden.py), stored in float32: the oracle must reproduce them, NaN and inf patterns
    included, to float32 rounding."""
    import os

    data = np.load(os.path.join(os.path.dirname(G.__file__), name + ".npz"))
    assert str(data["source"]).startswith("reference"), "regenerate the fixtures where the reference checkout exists"
    ans = G.answers(name)
    for key in ("out", "lse", "dq", "dk", "dv"):
        a = ans[key]
        if name.startswith("config1"):
            a = a[:, ::16] if key != "lse" else a[:, :, ::16]
        want = data[key]
        assert np.array_equal(np.isnan(a), np.isnan(want)), key
        ok = ~np.isnan(want)
        assert np.array_equal(np.isinf(a[ok]), np.isinf(want[ok])), key
        fin = ok & np.isfinite(want)
        if fin.any():  # (dK and dV of the random-segment case are NaN throughout, ring.py:146)
            scale = max(1.0, float(np.abs(want[fin]).max()))
            assert np.abs(a[fin] - want[fin]).max() <= 2e-7 * scale, key


def test_config1_ring_emulation_four_ranks():
    """The CPU-runnable configuration: 4 ranks, 256 rows each, causal, float32 block math."""
    q, k, v, do, extra = G.inputs("config1_causal_1024")
    fn = lambda **kw: O.self_attention_bias(True, **kw)
    qk = [{"q_positions": p} for p in O.shard(extra["q_pos"], 4)]
    kk = [{"kv_positions": p} for p in O.shard(extra["kv_pos"], 4)]
    qs, ks, vs, dos = (O.shard(x, 4) for x in (q, k, v, do))
    outs, lses = O.ring_attention_fwd(qs, ks, vs, fn, qk, kk, dtype=np.float32)
    dq, dk, dv = O.ring_attention_bwd(qs, ks, vs, outs, lses, dos, fn, qk, kk, dtype=np.float32)
    ans = G.answers("config1_causal_1024")
    np.testing.assert_allclose(O.unshard(outs), ans["out"], atol=2e-6)
    np.testing.assert_allclose(O.unshard(dq), ans["dq"], atol=2e-5)
    np.testing.assert_allclose(O.unshard(dk), ans["dk"], atol=2e-5)
    np.testing.assert_allclose(O.unshard(dv), ans["dv"], atol=2e-5)


def test_blas_block_port_equals_einsum_port():
    rng = np.random.default_rng(2)
    b, h, lq, lk, d = 2, 3, 20, 36, 8
    q, k, v, do = (rng.standard_normal((b, h, n, d)) for n in (lq, lk, lk, lq))
    bias = np.where(rng.random((b, 1, lq, lk)) < 0.3, -np.inf, 0.0)
    bias[:, :, 0] = -np.inf  # a fully masked row
    o0, m0, l0 = np.zeros((b, h, lq, d)), np.full((b, h, lq), -np.inf), np.zeros((b, h, lq))
    a = O.fwd_block(q, k, v, bias, o0, m0, l0, 0.3)
    c = O.fwd_block_mm(q, k, v, bias, o0, m0, l0, 0.3)
    for x, y in zip(a, c):
        np.testing.assert_allclose(x, y, atol=1e-12)
    out, L = O.finalize(*a)
    ga = O.bwd_block(q, k, v, bias, out, L, do, 0.3)
    gc = O.bwd_block_mm(q, k, v, bias, out, L, do, 0.3)
    for x, y in zip(ga, gc):
        np.testing.assert_allclose(x, y, atol=1e-12, equal_nan=True)
    assert O.timed_cpu_ring_causal(1, 2, 64, 8, 4) > 0
    assert O.causal_flops(1, 1, 4, 2) == 10 * 14 * 2
