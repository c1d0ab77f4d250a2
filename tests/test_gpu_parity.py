"""GPU parity tests: the CUDA engine, called through the C ABI, against the CPU oracle.

Shapes are those of the reference's tests (ring_attention/ring_test.py:49-52, 105-110,
177-182, 323-328) with NumPy-seeded inputs (JAX's PRNG stream cannot be regenerated).
Bounds: float32 1e-5 max-abs against the float64 oracle; bfloat16 2e-2 abs + 1e-2 rel
against the oracle evaluated on the bf16-rounded inputs.
"""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.golden import make_golden as G
from tests.util import check_close, make_inputs, to_dev

pytestmark = pytest.mark.gpu

FWD_SHAPES = [(0, 24, 16, 1, 2), (1, 128, 64, 4, 64), (2, 64, 512, 4, 16), (3, 2048, 2048, 4, 128)]
BWD_SHAPES = FWD_SHAPES[:3] + [(3, 128, 2048, 2, 128), (3, 2048, 128, 2, 128), (3, 2048, 2048, 4, 128)]
DTYPES = [torch.float32, torch.bfloat16]


def ra():
    import ring_attention_b200

    return ring_attention_b200


def _grads(fn, q, k, v, do):
    q, k, v = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = fn(q, k, v)
    (out.float() * do.float()).sum().backward()
    return out, q.grad, k.grad, v.grad


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed,lq,lk,h,d", BWD_SHAPES)
def test_ring_attention_single_rank_fwd_bwd(seed, lq, lk, h, d, dtype):
    """ring_test.py:45-171 with a ring of one: out and gradients equal dense attention."""
    q, k, v, do, _ = make_inputs(seed, 2, lq, lk, h, d, dtype)
    tq, tk, tv, tdo = (to_dev(x, dtype) for x in (q, k, v, do))
    out, dq, dk, dv = _grads(lambda a, b, c: ra().ring_attention(a, b, c, "sp", block_impl="simt"), tq, tk, tv, tdo)
    assert not torch.isnan(out).any()
    check_close(out, O.mha(q, k, v), dtype, "out")
    rq, rk, rv = O.mha_grads(q, k, v, do)
    big = lq * lk >= 2048 * 2048
    tol = 5e-5 if big else 1e-5  # 2048 float32 atomics per dq element at the largest shape
    check_close(dq, rq, dtype, "dq", tol)
    check_close(dk, rk, dtype, "dk", tol)
    check_close(dv, rv, dtype, "dv", tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed,lq,lk,h,d", FWD_SHAPES[:3] + [(3, 1024, 1024, 2, 128)])
def test_block_chain_equals_ring_of_eight(seed, lq, lk, h, d, dtype):
    """Eight chained block updates with carried (o, m, l) on one GPU reproduce what eight
    ranks compute (ring.py:104-137), and eight block VJPs sum to the dense gradients."""
    n = 8
    q, k, v, do, _ = make_inputs(seed, 2, lq, lk, h, d, dtype)
    scale = 1 / np.sqrt(d)
    bh = lambda x: to_dev(np.transpose(x, (0, 2, 1, 3)), dtype)
    tq, tdo = bh(q), bh(do)
    ks, vs = O.shard(k, n), O.shard(v, n)
    o = torch.zeros((2, h, lq, d), device="cuda")
    m = torch.full((2, h, lq), -float("inf"), device="cuda")
    l = torch.zeros((2, h, lq), device="cuda")
    for t in range(n):
        o, m, l = ra().fwd_block(tq, bh(ks[t]), bh(vs[t]), None, o, m, l, scale, block_impl="simt")
    out = o / l[..., None]
    L = m + torch.log(l)
    ref, ref_lse = O.mha(q, k, v, return_lse=True)
    check_close(out.permute(0, 2, 1, 3), ref, torch.float32, "out", 1e-5 if dtype == torch.float32 else 2e-2)
    check_close(L, ref_lse, torch.float32, "lse", 1e-5 if dtype == torch.float32 else 2e-2)
    # carried state against the oracle's own chain (ring.py:58-76)
    dq = torch.zeros((2, h, lq, d), device="cuda")
    dks, dvs = [], []
    out_in = out.to(dtype)
    for t in range(n):
        a, b_, c = ra().bwd_block(tq, bh(ks[t]), bh(vs[t]), None, out_in, L, tdo, scale, block_impl="simt")
        dq += a
        dks.append(b_)
        dvs.append(c)
    rq, rk, rv = O.mha_grads(q, k, v, do)
    check_close(dq.permute(0, 2, 1, 3), rq, dtype, "dq", 2e-5)
    check_close(torch.cat(dks, 2).permute(0, 2, 1, 3), rk, dtype, "dk", 2e-5)
    check_close(torch.cat(dvs, 2).permute(0, 2, 1, 3), rv, dtype, "dv", 2e-5)


@pytest.mark.parametrize("seed,lq,lk,h,d", FWD_SHAPES[:3])
def test_fwd_block_state_matches_oracle_step(seed, lq, lk, h, d):
    """One ra_fwd_block call against one oracle block update from a non-trivial state."""
    q, k, v, _, rng = make_inputs(seed, 2, lq, lk, h, d, torch.float32)
    bh = lambda x: np.ascontiguousarray(np.transpose(x, (0, 2, 1, 3)))
    qb, kb, vb = bh(q), bh(k), bh(v)
    bias = rng.standard_normal((2, h, lq, lk))
    bias[rng.random(bias.shape) < 0.3] = -np.inf
    o0 = rng.standard_normal((2, h, lq, d))
    m0 = rng.standard_normal((2, h, lq))
    m0[rng.random(m0.shape) < 0.2] = -np.inf
    l0 = rng.random((2, h, lq)) + 0.5
    o0[np.isneginf(m0)] = 0
    l0[np.isneginf(m0)] = 0
    want = O.fwd_block(qb, kb, vb, bias, o0, m0, l0, 0.37)
    got = ra().fwd_block(to_dev(qb), to_dev(kb), to_dev(vb), to_dev(bias), to_dev(o0), to_dev(m0), to_dev(l0), 0.37,
                         block_impl="simt")
    for g, w, name in zip(got, want, "oml"):
        check_close(g, w, torch.float32, name, 2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed,lq,lk,h,d", FWD_SHAPES[:3] + [(3, 1024, 1024, 2, 128)])
def test_ring_attention_bias_fn_nan_pattern(seed, lq, lk, h, d, dtype):
    """ring_test.py:174-300: a user bias_fn over independent random segment ids; rows that
    see no key are NaN exactly where dense softmax is, and gradients match."""
    q, k, v, do, rng = make_inputs(seed, 2, lq, lk, h, d, dtype)
    qseg = rng.integers(0, max(lq // 5, 1), (2, lq)).astype(np.int32)
    kseg = rng.integers(0, max(lq // 5, 1), (2, lk)).astype(np.int32)
    bias = np.where(qseg[:, :, None] == kseg[:, None, :], 0.0, -np.inf)[:, None].repeat(h, 1)

    def bias_fn(q_segment_ids, kv_segment_ids):
        mask = q_segment_ids[:, :, None] == kv_segment_ids[:, None, :]
        z = torch.zeros(mask.shape, device=mask.device)
        return torch.where(mask, z, z - float("inf"))[:, None].expand(-1, h, -1, -1)

    tq, tk, tv, tdo = (to_dev(x, dtype) for x in (q, k, v, do))
    kw = dict(bias_q_kwargs={"q_segment_ids": to_dev(qseg, torch.int32)},
              bias_kv_kwargs={"kv_segment_ids": to_dev(kseg, torch.int32)})
    ref = O.mha(q, k, v, bias)
    rq, rk, rv = O.mha_grads(q, k, v, do, bias)
    # dense-tile path (reference NaN semantics); the compiled-in segment mask, whose backward by
    # default gives rows that saw no key a zero contribution instead of NaN; and the same mask
    # with strict_nan, which reproduces the reference's NaN pattern (ring.py:146, ring_test.py:273)
    for fn, nan in ((bias_fn, "match"), (ra().ScoreMod(), "finite"), (ra().ScoreMod(strict_nan=True), "match")):
        out, dq, dk, dv = _grads(lambda a, b, c: ra().ring_attention(a, b, c, "sp", bias_fn=fn, block_impl="simt", **kw),
                                 tq, tk, tv, tdo)
        check_close(out, ref, dtype, "out")
        check_close(dq, rq, dtype, "dq", 2e-5, nan=nan)
        check_close(dk, rk, dtype, "dk", 2e-5, nan=nan)
        check_close(dv, rv, dtype, "dv", 2e-5, nan=nan)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed,length,h,d", [(0, 16, 1, 2), (1, 128, 4, 64), (2, 512, 4, 16), (4, 2048, 4, 64)])
def test_ring_self_attention(seed, length, h, d, dtype):
    """ring_test.py:320-378: causal + random segment ids through ring_self_attention."""
    q, k, v, do, rng = make_inputs(seed, 2, length, length, h, d, dtype)
    seg = rng.integers(0, 5, (2, length)).astype(np.int32)
    pos = np.broadcast_to(np.arange(length, dtype=np.int32), (2, length)).copy()
    i = np.arange(length)
    mask = (seg[:, :, None] == seg[:, None, :]) & (i[None, :] <= i[:, None])
    bias = np.where(mask, 0.0, -np.inf)[:, None]
    tq, tk, tv, tdo = (to_dev(x, dtype) for x in (q, k, v, do))
    fn = lambda a, b, c: ra().ring_self_attention(
        a, b, c, None, ra().PartitionSpec(None, "sp"), causal=True,
        segment_ids=to_dev(seg, torch.int32), positions=to_dev(pos, torch.int32), block_impl="simt")
    out, dq, dk, dv = _grads(fn, tq, tk, tv, tdo)
    check_close(out, O.mha(q, k, v, bias), dtype, "out")
    rq, rk, rv = O.mha_grads(q, k, v, do, bias)
    check_close(dq, rq, dtype, "dq", 2e-5)
    check_close(dk, rk, dtype, "dk", 2e-5)
    check_close(dv, rv, dtype, "dv", 2e-5)


MODS = [
    dict(causal=True), dict(causal=True, seg=True), dict(seg=True), dict(seg=True, prefix=True),
    dict(prefix=True), dict(causal=True, alibi=True), dict(causal=True, alibi=True, window=37),
    dict(causal=True, window=100), dict(window=64),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mod", MODS, ids=lambda m: "+".join(sorted(m)))
def test_score_mod_variants_match_dense_bias(mod, dtype):
    """Every compiled-in score-mod against the oracle's dense bias for the same rule, with
    shuffled (non-contiguous) positions so that nothing depends on block indices."""
    b, h, lq, lk, d = 2, 4, 192, 320, 64
    q, k, v, do, rng = make_inputs(7, b, lq, lk, h, d, dtype)
    kpos = np.stack([rng.permutation(lk) for _ in range(b)]).astype(np.int32)
    qpos = np.stack([rng.permutation(lk)[:lq] for _ in range(b)]).astype(np.int32)
    qpos[:, 0] = lk - 1  # at least one row sees every causal key
    seg = mod.get("seg")
    qseg = rng.integers(0, 3, (b, lq)).astype(np.int32) if seg else None
    kseg = rng.integers(0, 3, (b, lk)).astype(np.int32) if seg else None
    qpre = rng.integers(0, 2, (b, lq)).astype(bool) if mod.get("prefix") else None
    kpre = rng.integers(0, 2, (b, lk)).astype(bool) if mod.get("prefix") else None
    slopes = O.alibi_slopes(h) if mod.get("alibi") else None
    bias = O.score_mod_bias(b, h, qpos, kpos, qseg, kseg, qpre, kpre, mod.get("causal", False), slopes,
                            mod.get("window", 0))
    T = lambda a, t=torch.int32: None if a is None else to_dev(a, t)
    sm = ra().ScoreMod(causal=mod.get("causal", False), alibi_slopes=T(slopes, torch.float32),
                       window=mod.get("window", 0))
    qkw = {"q_positions": T(qpos), "q_segment_ids": T(qseg), "q_prefix_mask": T(qpre, torch.bool)}
    kkw = {"kv_positions": T(kpos), "kv_segment_ids": T(kseg), "kv_prefix_mask": T(kpre, torch.bool)}
    tq, tk, tv, tdo = (to_dev(x, dtype) for x in (q, k, v, do))
    out, dq, dk, dv = _grads(lambda a, b_, c: ra().ring_attention(a, b_, c, "sp", bias_fn=sm, bias_q_kwargs=qkw,
                                                                 bias_kv_kwargs=kkw, block_impl="simt"), tq, tk, tv, tdo)
    check_close(out, O.mha(q, k, v, bias), dtype, "out")
    rq, rk, rv = O.mha_grads(q, k, v, do, bias)
    # shuffled positions leave some rows without any visible key: see check_close
    check_close(dq, rq, dtype, "dq", 2e-5, nan="finite")
    check_close(dk, rk, dtype, "dk", 2e-5, nan="finite")
    check_close(dv, rv, dtype, "dv", 2e-5, nan="finite")
    # the same call with the reference's NaN semantics switched on: the pattern must match exactly
    sm.strict_nan = True
    out, dq, dk, dv = _grads(lambda a, b_, c: ra().ring_attention(a, b_, c, "sp", bias_fn=sm, bias_q_kwargs=qkw,
                                                                 bias_kv_kwargs=kkw, block_impl="simt"), tq, tk, tv, tdo)
    check_close(dq, rq, dtype, "dq strict", 2e-5)
    check_close(dk, rk, dtype, "dk strict", 2e-5)
    check_close(dv, rv, dtype, "dv strict", 2e-5)


@pytest.mark.parametrize("name", list(G.CASES))
def test_golden_fixtures(name):
    """The committed fixtures (tests/golden/*.npz), float32 engine."""
    seed, b, lq, lk, h, d, n, mask = G.CASES[name]
    q, k, v, do, extra = G.inputs(name)
    data = np.load(os.path.join(os.path.dirname(G.__file__), name + ".npz"))
    T = lambda a: to_dev(a, torch.int32)
    sm, qkw, kkw = None, None, None
    if mask != "none":
        sm = ra().ScoreMod(causal="causal" in mask)
        qkw = {"q_positions": T(extra["q_pos"]) if "q_pos" in extra else None,
               "q_segment_ids": T(extra["q_seg"]) if "q_seg" in extra else None,
               "q_prefix_mask": to_dev(extra["q_pre"], torch.bool) if "q_pre" in extra else None}
        kkw = {"kv_positions": T(extra["kv_pos"]) if "kv_pos" in extra else None,
               "kv_segment_ids": T(extra["kv_seg"]) if "kv_seg" in extra else None,
               "kv_prefix_mask": to_dev(extra["kv_pre"], torch.bool) if "kv_pre" in extra else None}
    tq, tk, tv, tdo = (to_dev(x) for x in (q, k, v, do))
    out, dq, dk, dv = _grads(lambda a, b_, c: ra().ring_attention(a, b_, c, "sp", bias_fn=sm, bias_q_kwargs=qkw,
                                                                 bias_kv_kwargs=kkw, block_impl="simt"), tq, tk, tv, tdo)
    sub = (lambda t: t[:, ::16]) if name.startswith("config1") else (lambda t: t)
    nan = "match" if mask == "none" else "finite"
    check_close(sub(out), data["out"], torch.float32, "out", 1e-5)
    check_close(sub(dq), data["dq"], torch.float32, "dq", 2e-5, nan=nan)
    check_close(sub(dk), data["dk"], torch.float32, "dk", 2e-5, nan=nan)
    check_close(sub(dv), data["dv"], torch.float32, "dv", 2e-5, nan=nan)


def test_different_value_head_dim_and_strided_inputs():
    """dv != dk (the reference's Pallas path hard-codes dk, ring_kernel.py:170) and inputs
    that are views with gaps between rows."""
    b, lq, lk, h, d, dv = 2, 70, 90, 3, 24, 40
    q, k, v, do, _ = make_inputs(3, b, lq, lk, h, d, torch.float32, dv=dv)
    pad = lambda x: to_dev(np.concatenate([x, np.zeros_like(x)], -1))[..., : x.shape[-1]]
    tq, tk, tv, tdo = pad(q), pad(k), pad(v), to_dev(do)
    assert not tq.is_contiguous()
    out, dq, dk, dvv = _grads(lambda a, b_, c: ra().ring_attention(a, b_, c, "sp", block_impl="simt"), tq, tk, tv, tdo)
    check_close(out, O.mha(q, k, v), torch.float32, "out")
    rq, rk, rv = O.mha_grads(q, k, v, do)
    check_close(dq, rq, torch.float32, "dq")
    check_close(dk, rk, torch.float32, "dk")
    check_close(dvv, rv, torch.float32, "dv")


def test_launches_are_counted_and_native():
    from ring_attention_b200._lib import lib

    before = lib.ra_launch_count()
    q = torch.randn(1, 64, 2, 32, device="cuda")
    ra().ring_attention(q, q, q, "sp", block_impl="simt")
    assert lib.ra_launch_count() >= before + 2
    assert lib.ra_last_impl() == 1
