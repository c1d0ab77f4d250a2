"""The oracle against the reference's own code.

JAX cannot be installed here, so the reference's ring.py is run on a NumPy stand-in for the
handful of JAX names it uses (tests/golden/jax_on_numpy.py: one thread per virtual device,
`ppermute` / `psum` at a barrier, `scan` as a loop, `custom_vjp` as a tape).  Everything else
that executes is the reference's Python: `ring_attention`, `ring_self_attention`, the custom-VJP
forward and backward scans, `_fwd_block` / `_bwd_block`, `_rotate_block` and the built-in mask
builder, in float64.  Needs the reference checkout; skipped where it is absent.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

import reference_run as R  # noqa: E402
from oracle import oracle as O  # noqa: E402

pytestmark = pytest.mark.skipif(not R.available(), reason="the reference checkout is not on this machine")


def _same(name, got, want, tol=1e-11):
    assert got.shape == want.shape, (name, got.shape, want.shape)
    assert np.array_equal(np.isnan(got), np.isnan(want)), f"{name}: NaN pattern differs"
    ok = ~np.isnan(want)
    assert np.array_equal(np.isinf(got[ok]), np.isinf(want[ok])), f"{name}: inf pattern differs"
    fin = ok & np.isfinite(want)
    err = np.abs(got[fin] - want[fin]).max() if fin.any() else 0.0
    assert err <= tol, f"{name}: max abs difference {err:.3e}"


def _compare(ans, q, k, v, do, bias):
    out, lse = O.mha(q, k, v, bias, return_lse=True)
    dq, dk, dv = O.mha_grads(q, k, v, do, bias)
    for name, want in (("out", out), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        _same(name, ans[name], want)


# ring_test.py:49-52 and :105-110: (q_len, kv_len, heads, head dim), 8 devices, batch 2
@pytest.mark.parametrize("lq,lk,h,d", [(24, 16, 1, 2), (128, 64, 4, 64), (64, 128, 2, 16), (8, 8, 1, 1)])
def test_general_entry_point_plain_and_cross_attention(lq, lk, h, d):
    rng = np.random.default_rng(lq + lk)
    q, k, v, do = (rng.standard_normal((2, n, h, d)) for n in (lq, lk, lk, lq))
    ans = R.reference_answers(q, k, v, do, 8)
    _compare(ans, q, k, v, do, None)
    # the oracle's own ring over 8 virtual ranks (its restatement of the schedule) against the same run
    sh = lambda x: np.split(x, 8, axis=1)
    out, res = O.ring_attention_fwd(sh(q), sh(k), sh(v))
    _same("ring out", np.concatenate(out, axis=1), ans["out"])


def test_general_entry_point_with_a_segment_bias_fn():
    """Independent random ids for queries and keys (ring_test.py:203-208): some query rows see
    no key at all, and the reference's NaN pattern must be reproduced."""
    rng = np.random.default_rng(3)
    b, lq, lk, h, d = 2, 128, 64, 4, 16
    q, k, v, do = (rng.standard_normal((b, n, h, d)) for n in (lq, lk, lk, lq))
    q_seg = rng.integers(0, lq // 5, (b, lq)).astype(np.int32)
    kv_seg = rng.integers(0, lq // 5, (b, lk)).astype(np.int32)
    ans = R.reference_answers(q, k, v, do, 8, q_seg=q_seg, kv_seg=kv_seg)
    bias = O.score_mod_bias(b, h, q_segment_ids=q_seg, kv_segment_ids=kv_seg)
    assert np.isnan(ans["out"]).any(), "this case is meant to have fully masked rows"
    _compare(ans, q, k, v, do, bias)


# (no mask at all is left out: the reference's mask builder then indexes a 0-d bias, ring.py:409)
@pytest.mark.parametrize("causal,segments,prefix", [(True, False, False), (True, True, False), (False, True, False),
                                                     (False, False, True), (False, True, True)])
def test_self_attention_entry_point_and_its_mask_builder(causal, segments, prefix):
    """ring_self_attention (ring.py:328-449) through the stand-in's shard_map: bidirectional,
    block-sparse, causal and prefix-LM masks and their combinations (ring_test.py:323-350)."""
    rng = np.random.default_rng(11)
    b, l, h, d, n = 2, 64, 2, 8, 8
    q, k, v, do = (rng.standard_normal((b, l, h, d)) for _ in range(4))
    seg = np.sort(rng.integers(0, 5, (b, l)), axis=1).astype(np.int32) if segments else None
    pos = np.broadcast_to(np.arange(l, dtype=np.int32), (b, l)).copy() if (causal or prefix) else None
    pre = (np.arange(l)[None] < rng.integers(4, 40, (b, 1))) if prefix else None
    ans = R.reference_answers(q, k, v, do, n, q_seg=seg, kv_seg=seg, q_pos=pos, kv_pos=pos, q_pre=pre, kv_pre=pre,
                              causal=causal, api="ring_self_attention")
    bias = O.score_mod_bias(b, h, q_positions=pos, kv_positions=pos, q_segment_ids=seg, kv_segment_ids=seg,
                            q_prefix_mask=pre, kv_prefix_mask=pre, causal=causal)
    _compare(ans, q, k, v, do, bias)


def test_block_functions_directly():
    """_fwd_block / _bwd_block (ring.py:58-76, 140-157) against the oracle's block math, with a
    carried state and a bias that masks some rows entirely."""
    ref = R.load_reference()
    rng = np.random.default_rng(5)
    b, h, lq, lk, d = 2, 3, 12, 20, 4
    q, k, v, do = (rng.standard_normal(s) for s in ((b, h, lq, d), (b, h, lk, d), (b, h, lk, d), (b, h, lq, d)))
    bias = np.where(rng.random((b, 1, lq, lk)) < 0.4, -np.inf, 0.0)
    bias[:, :, 3] = -np.inf
    o0 = rng.standard_normal((b, h, lq, d))
    m0 = rng.standard_normal((b, h, lq))
    m0[:, :, 5] = -np.inf
    l0 = rng.random((b, h, lq)) + 0.5
    got = ref._fwd_block(q, k, v, bias, o0, m0, l0, 0.37)
    want = O.fwd_block(q, k, v, bias, o0, m0, l0, 0.37)
    for name, g, w in zip(("o", "m", "l"), got, want):
        _same(name, np.asarray(g), w)
    L = rng.standard_normal((b, h, lq)) + 3
    got = ref._bwd_block(q, k, v, bias, o0, L, do, 0.37)
    want = O.bwd_block(q, k, v, bias, o0, L, do, 0.37)
    for name, g, w in zip(("dq", "dk", "dv"), got, want):
        _same(name, np.asarray(g), w)


# ---- the Pallas kernels of ring_kernel.py, through the stand-in's interpreter of the Pallas calls
# they make (float32, as the reference's own tests run them; m and l are float32 inside the kernels)
def _compare32(ans, q, k, v, do, bias, tol=2e-5):
    out, lse = O.mha(q, k, v, bias, return_lse=True)
    dq, dk, dv = O.mha_grads(q, k, v, do, bias)
    for name, want in (("out", out), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        _same(name, ans[name].astype(np.float64), want, tol)


@pytest.mark.parametrize("lq,lk,h,d", [(24, 16, 1, 2), (128, 64, 4, 64), (2048, 1024, 2, 16)])
def test_pallas_kernels_plain_and_cross_attention(lq, lk, h, d):
    """ring_test.py:49-52, 105-110 with block_impl="pallas": 3-row shards up to two query tiles
    per device."""
    rng = np.random.default_rng(lq)
    q, k, v, do = (rng.standard_normal((2, n, h, d)).astype(np.float32) for n in (lq, lk, lk, lq))
    ans = R.reference_answers(q, k, v, do, 8, block_impl="pallas", dtype=np.float32)
    _compare32(ans, q, k, v, do, None)


def test_pallas_kernels_with_the_built_in_mask_and_two_key_tiles_per_device():
    """Causal + segments self attention, 256 tokens per device: two query tiles and two key
    tiles per block call, the bias tile read through ring_kernel.py:253-256."""
    rng = np.random.default_rng(21)
    b, l, h, d, n = 1, 2048, 2, 16, 8
    q, k, v, do = (rng.standard_normal((b, l, h, d)).astype(np.float32) for _ in range(4))
    seg = np.sort(rng.integers(0, 5, (b, l)), axis=1).astype(np.int32)
    pos = np.broadcast_to(np.arange(l, dtype=np.int32), (b, l)).copy()
    ans = R.reference_answers(q, k, v, do, n, q_seg=seg, kv_seg=seg, q_pos=pos, kv_pos=pos, causal=True,
                              api="ring_self_attention", block_impl="pallas", dtype=np.float32)
    bias = O.score_mod_bias(b, h, q_positions=pos, kv_positions=pos, q_segment_ids=seg, kv_segment_ids=seg, causal=True)
    _compare32(ans, q, k, v, do, bias)


def test_pallas_kernels_with_a_segment_bias_fn_keep_the_nan_pattern():
    rng = np.random.default_rng(3)
    b, lq, lk, h, d = 2, 128, 64, 2, 16
    q, k, v, do = (rng.standard_normal((b, n, h, d)).astype(np.float32) for n in (lq, lk, lk, lq))
    q_seg = rng.integers(0, lq // 5, (b, lq)).astype(np.int32)
    kv_seg = rng.integers(0, lq // 5, (b, lk)).astype(np.int32)
    ans = R.reference_answers(q, k, v, do, 8, q_seg=q_seg, kv_seg=kv_seg, block_impl="pallas", dtype=np.float32)
    bias = O.score_mod_bias(b, h, q_segment_ids=q_seg, kv_segment_ids=kv_seg)
    assert np.isnan(ans["out"]).any()
    _compare32(ans, q, k, v, do, bias)


def test_zigzag_token_layout_is_legal_in_the_reference():
    """The masks are driven by the position arrays (ring.py:396), not by block indices, so the
    reference itself gives the same answer when every device holds chunks r and 2N-1-r of the
    sequence (the load-balanced layout the benchmark uses) instead of one contiguous chunk."""
    from ring_attention_b200.layout import zigzag_indices

    rng = np.random.default_rng(8)
    b, l, h, d, n = 2, 128, 2, 8, 4
    q, k, v, do = (rng.standard_normal((b, l, h, d)) for _ in range(4))
    seg = np.sort(rng.integers(0, 3, (b, l)), axis=1).astype(np.int32)
    pos = np.broadcast_to(np.arange(l, dtype=np.int32), (b, l)).copy()
    order = np.concatenate([zigzag_indices(l, r, n).numpy() for r in range(n)])  # device r's tokens, in rank order
    take = lambda x: np.ascontiguousarray(x[:, order])
    ans = R.reference_answers(take(q), take(k), take(v), take(do), n, q_seg=take(seg), kv_seg=take(seg),
                              q_pos=take(pos), kv_pos=take(pos), causal=True, api="ring_self_attention")
    bias = O.score_mod_bias(b, h, q_positions=pos, kv_positions=pos, q_segment_ids=seg, kv_segment_ids=seg, causal=True)
    out, lse = O.mha(q, k, v, bias, return_lse=True)
    dq, dk, dv = O.mha_grads(q, k, v, do, bias)
    back = np.argsort(order)
    for name, want in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        _same(name, ans[name][:, back], want)
    _same("lse", ans["lse"][:, :, back], lse)


@pytest.mark.parametrize("seed", range(12))
def test_random_small_cases(seed):
    """Seeded random shapes, device counts and mask combinations, both block implementations."""
    rng = np.random.default_rng(1000 + seed)
    n = int(rng.choice([2, 3, 4, 8]))
    c = int(rng.choice([1, 3, 8, 16]))
    b, h, d = int(rng.integers(1, 3)), int(rng.integers(1, 4)), int(rng.choice([1, 2, 8, 16]))
    l = n * c
    impl = "pallas" if seed % 2 else "jax"
    dtype = np.float32 if impl == "pallas" else np.float64
    q, k, v, do = (rng.standard_normal((b, l, h, d)).astype(dtype) for _ in range(4))
    kind = seed % 4
    causal = kind in (0, 1)
    seg = np.sort(rng.integers(0, 3, (b, l)), axis=1).astype(np.int32) if kind in (1, 2, 3) else None
    pre = (np.arange(l)[None] < rng.integers(1, l + 1, (b, 1))) if kind == 3 else None
    pos = np.broadcast_to(np.arange(l, dtype=np.int32), (b, l)).copy() if (causal or pre is not None) else None
    ans = R.reference_answers(q, k, v, do, n, q_seg=seg, kv_seg=seg, q_pos=pos, kv_pos=pos, q_pre=pre, kv_pre=pre,
                              causal=causal, api="ring_self_attention", block_impl=impl, dtype=dtype)
    bias = O.score_mod_bias(b, h, q_positions=pos, kv_positions=pos, q_segment_ids=seg, kv_segment_ids=seg,
                            q_prefix_mask=pre, kv_prefix_mask=pre, causal=causal)
    if impl == "pallas":
        _compare32(ans, q, k, v, do, bias)
    else:
        _compare(ans, q, k, v, do, bias)
