"""GPU parity tests of the tcgen05 (bf16 tensor-core) block kernels against the CPU oracle.

Same bound as every bf16 test: 2e-2 abs + 1e-2 rel against the float64 oracle evaluated on
the bf16-rounded inputs.  `block_impl="tcgen05"` makes the call fail instead of falling
back when a shape does not fit the tensor-core kernels.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import check_close, make_inputs, to_dev

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def ra():
    import ring_attention_b200

    return ring_attention_b200


def _status_clean():
    from ring_attention_b200._lib import lib

    bits = C.c_uint32(0)
    assert lib.ra_device_status(C.byref(bits)) == 0, hex(bits.value)


def _grads(fn, q, k, v, do):
    q, k, v = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = fn(q, k, v)
    out.backward(do)
    return out, q.grad, k.grad, v.grad


@pytest.mark.parametrize("b,h,lq,lk,d", [(1, 1, 128, 128, 128), (2, 2, 384, 640, 128), (1, 2, 256, 512, 64),
                                          (2, 3, 512, 128, 64), (1, 4, 2048, 2048, 128)])
def test_fwd_block_state(b, h, lq, lk, d):
    """(o, m, l) after one call and after a chain of calls with carried state (ring.py:58-76)."""
    q, k, v, _, _ = make_inputs(1, b, lq, lk, h, d, BF)
    bh = lambda x: np.ascontiguousarray(np.transpose(x, (0, 2, 1, 3)))
    qb, kb, vb = bh(q), bh(k), bh(v)
    scale = 1 / np.sqrt(d)
    cut = [(lk // 256) * 128] if lk >= 256 else []  # two K/V blocks, each a multiple of 128 rows
    o = torch.zeros((b, h, lq, d), device="cuda")
    m = torch.full((b, h, lq), -float("inf"), device="cuda")
    l = torch.zeros((b, h, lq), device="cuda")
    oo, mm, ll = np.zeros((b, h, lq, d)), np.full((b, h, lq), -np.inf), np.zeros((b, h, lq))
    for kc, vc in zip(np.split(kb, cut, 2), np.split(vb, cut, 2)):
        o, m, l = ra().fwd_block(to_dev(qb, BF), to_dev(kc, BF), to_dev(vc, BF), None, o, m, l, scale,
                                 block_impl="tcgen05")
        oo, mm, ll = O.fwd_block(qb, kc, vc, None, oo, mm, ll, scale)
    _status_clean()
    check_close(m, mm, torch.float32, "m", 1e-4)
    check_close(l / to_dev(ll), np.ones_like(ll), torch.float32, "l (relative)", 2e-3)
    check_close(o / l[..., None], oo / ll[..., None], BF, "o / l")


MODS = [
    dict(causal=True), dict(causal=True, seg=True), dict(seg=True), dict(seg=True, prefix=True),
    dict(prefix=True), dict(causal=True, alibi=True), dict(causal=True, alibi=True, window=300), dict(alibi=True),
    dict(causal=True, window=200), dict(window=256),
]


@pytest.mark.parametrize("layout", ["contiguous", "shuffled", "sorted-docs"])
@pytest.mark.parametrize("mod", MODS, ids=lambda m: "+".join(sorted(m)))
def test_score_mods_forward(mod, layout):
    """Every compiled-in score-mod on the tensor-core path, with positions in order (tile
    skipping active), shuffled (every tile mixed) and with sorted document ids."""
    b, h, lq, lk, d = 2, 2, 512, 768, 128
    q, k, v, do, rng = make_inputs(9, b, lq, lk, h, d, BF)
    if layout == "shuffled":
        kpos = np.stack([rng.permutation(lk) for _ in range(b)]).astype(np.int32)
        qpos = np.stack([rng.permutation(lk)[:lq] for _ in range(b)]).astype(np.int32)
        qpos[:, 0] = lk - 1
    else:
        kpos = np.broadcast_to(np.arange(lk, dtype=np.int32), (b, lk)).copy()
        qpos = np.broadcast_to(np.arange(lk - lq, lk, dtype=np.int32), (b, lq)).copy()
    qseg = kseg = qpre = kpre = None
    if mod.get("seg"):
        if layout == "sorted-docs":
            kseg = np.sort(rng.integers(0, 4, (b, lk)), axis=1).astype(np.int32)
            qseg = kseg[:, lk - lq:].copy()
        else:
            kseg = rng.integers(0, 3, (b, lk)).astype(np.int32)
            qseg = rng.integers(0, 3, (b, lq)).astype(np.int32)
            qseg[:, 0] = kseg[:, 0]
    if mod.get("prefix"):
        kpre = (np.arange(lk)[None] < 200).repeat(b, 0) if layout != "shuffled" else rng.integers(0, 2, (b, lk)).astype(bool)
        qpre = kpre[:, lk - lq:].copy() if layout != "shuffled" else rng.integers(0, 2, (b, lq)).astype(bool)
    slopes = O.alibi_slopes(h) if mod.get("alibi") else None
    bias = O.score_mod_bias(b, h, qpos, kpos, qseg, kseg, qpre, kpre, mod.get("causal", False), slopes,
                            mod.get("window", 0))
    T = lambda a, t=torch.int32: None if a is None else to_dev(a, t)
    sm = ra().ScoreMod(causal=mod.get("causal", False), alibi_slopes=T(slopes, torch.float32), window=mod.get("window", 0))
    qkw = {"q_positions": T(qpos), "q_segment_ids": T(qseg), "q_prefix_mask": T(qpre, torch.bool)}
    kkw = {"kv_positions": T(kpos), "kv_segment_ids": T(kseg), "kv_prefix_mask": T(kpre, torch.bool)}
    tq, tk, tv, tdo = (to_dev(x, BF) for x in (q, k, v, do))
    out, dq, dk, dv = _grads(lambda a, b_, c: ra().ring_attention(a, b_, c, "sp", bias_fn=sm, bias_q_kwargs=qkw,
                                                                 bias_kv_kwargs=kkw, block_impl="tcgen05"), tq, tk, tv, tdo)
    _status_clean()
    check_close(out, O.mha(q, k, v, bias), BF, "out")
    rq, rk, rv = O.mha_grads(q, k, v, do, bias)
    check_close(dq, rq, BF, "dq", nan="finite")
    check_close(dk, rk, BF, "dk", nan="finite")
    check_close(dv, rv, BF, "dv", nan="finite")
    # with the reference's NaN semantics switched on the NaN pattern matches exactly (ring.py:146)
    sm.strict_nan = True
    out, dq, dk, dv = _grads(lambda a, b_, c: ra().ring_attention(a, b_, c, "sp", bias_fn=sm, bias_q_kwargs=qkw,
                                                                 bias_kv_kwargs=kkw, block_impl="tcgen05"), tq, tk, tv, tdo)
    _status_clean()
    check_close(dq, rq, BF, "dq strict")
    check_close(dk, rk, BF, "dk strict")
    check_close(dv, rv, BF, "dv strict")


@pytest.mark.parametrize("seed,lq,lk,h,d", [(1, 128, 2048, 2, 128), (3, 2048, 128, 2, 128), (3, 2048, 2048, 4, 128),
                                             (4, 2048, 2048, 4, 64), (5, 640, 896, 3, 64)])
def test_ring_of_one_fwd_bwd(seed, lq, lk, h, d):
    """ring_test.py:105-110 shapes that fit the tensor-core kernels: out and gradients."""
    q, k, v, do, _ = make_inputs(seed, 2, lq, lk, h, d, BF)
    tq, tk, tv, tdo = (to_dev(x, BF) for x in (q, k, v, do))
    out, dq, dk, dv = _grads(lambda a, b, c: ra().ring_attention(a, b, c, "sp", block_impl="tcgen05"), tq, tk, tv, tdo)
    _status_clean()
    from ring_attention_b200._lib import lib

    assert lib.ra_last_impl() == 2
    check_close(out, O.mha(q, k, v), BF, "out")
    rq, rk, rv = O.mha_grads(q, k, v, do)
    check_close(dq, rq, BF, "dq")
    check_close(dk, rk, BF, "dk")
    check_close(dv, rv, BF, "dv")


def test_emulated_ring_of_eight_causal_with_state():
    """Eight block calls with carried state and per-chunk position offsets reproduce a causal
    ring of eight ranks (the cross-device block offsets come from the position arrays)."""
    n, b, h, c, d = 8, 1, 2, 256, 128
    S = n * c
    q, k, v, do, _ = make_inputs(2, b, S, S, h, d, BF)
    pos = np.broadcast_to(np.arange(S, dtype=np.int32), (b, S))
    bias = O.score_mod_bias(b, h, pos, pos, causal=True)
    ref, ref_lse = O.mha(q, k, v, bias, return_lse=True)
    from ring_attention_b200 import _lib
    from ring_attention_b200._lib import RaScoreMod, RaShape, RaTensor, check, lib

    check(lib.ra_set_impl(_lib.RA_IMPL_TCGEN05))
    rank = 5  # the rank whose rows are checked
    sl = slice(rank * c, (rank + 1) * c)
    tq = to_dev(q[:, sl], BF)
    qpos = to_dev(pos[:, sl], torch.int32)
    o = torch.empty((b, h, c, d), device="cuda")
    m = torch.empty((b, h, c), device="cuda")
    l = torch.empty((b, h, c), device="cuda")
    sh = RaShape(b, h, c, c, d, d, _lib.RA_DTYPE_BF16, 1 / np.sqrt(d))
    tv_ = lambda t: C.byref(RaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)))
    for t in range(n):
        src = lib.ra_ring_source(rank, n, t)
        ks = slice(src * c, (src + 1) * c)
        tk, tvv, kpos = to_dev(k[:, ks], BF), to_dev(v[:, ks], BF), to_dev(pos[:, ks], torch.int32)
        mod = RaScoreMod()
        mod.kinds = _lib.RA_MOD_CAUSAL
        mod.q_pos, mod.kv_pos = qpos.data_ptr(), kpos.data_ptr()
        check(lib.ra_fwd_block(C.byref(sh), tv_(tq), tv_(tk), tv_(tvv), C.byref(mod), o.data_ptr(), m.data_ptr(),
                               l.data_ptr(), int(t == 0), None))
        torch.cuda.synchronize()
    _status_clean()
    out = (o / l[..., None]).permute(0, 2, 1, 3)
    check_close(out, ref[:, sl], BF, "out")
    check_close(m + torch.log(l), ref_lse[:, :, sl], torch.float32, "lse", 2e-3)


@pytest.mark.parametrize("seed,lq,lk,h,d,head_bias", [(3, 1024, 1024, 2, 128, True), (5, 640, 896, 3, 64, False),
                                                       (6, 256, 384, 2, 128, True)])
def test_bias_fn_callable_runs_on_the_tensor_core_kernels(seed, lq, lk, h, d, head_bias):
    """ring_test.py:174-300 on the tcgen05 path: any callable's dense bias tile (ring.py:107) is
    added inside the tensor-core kernels; rows that see no key are NaN exactly where dense
    softmax is (ring_test.py:273), and so are the gradients they poison (ring.py:146)."""
    from ring_attention_b200._lib import RA_IMPL_TCGEN05, lib

    q, k, v, do, rng = make_inputs(seed, 2, lq, lk, h, d, BF)
    qseg = rng.integers(0, max(lq // 5, 1), (2, lq)).astype(np.int32)
    kseg = rng.integers(0, max(lq // 5, 1), (2, lk)).astype(np.int32)
    qseg[:, 5] = 10 ** 6  # a query row that no key shares a segment with
    extra = rng.standard_normal((2, h if head_bias else 1, lq, lk)) * 0.5  # a real additive term, not only a mask
    bias = np.where((qseg[:, :, None] == kseg[:, None, :])[:, None], extra, -np.inf)
    bias = np.broadcast_to(bias, (2, h, lq, lk))
    tex = to_dev(extra, torch.float32)

    def bias_fn(q_segment_ids, kv_segment_ids):
        mask = (q_segment_ids[:, :, None] == kv_segment_ids[:, None, :])[:, None]
        return torch.where(mask, tex, torch.full_like(tex, float("-inf")))  # [b, h or 1, lq, lk]

    tq, tk, tv, tdo = (to_dev(x, BF) for x in (q, k, v, do))
    kw = dict(bias_q_kwargs={"q_segment_ids": to_dev(qseg, torch.int32)},
              bias_kv_kwargs={"kv_segment_ids": to_dev(kseg, torch.int32)})
    out, dq, dk, dv = _grads(lambda a, b, c: ra().ring_attention(a, b, c, "sp", bias_fn=bias_fn, block_impl="tcgen05", **kw),
                             tq, tk, tv, tdo)
    assert lib.ra_last_impl() == RA_IMPL_TCGEN05
    _status_clean()
    ref = O.mha(q, k, v, bias)
    rq, rk, rv = O.mha_grads(q, k, v, do, bias)
    assert np.isnan(ref).any(), "the case should have rows that see no key"
    check_close(out, ref, BF, "out")
    check_close(dq, rq, BF, "dq")
    check_close(dk, rk, BF, "dk")
    check_close(dv, rv, BF, "dv")
