"""CPU tests of the host side: the C-ABI library loads and exports what the header
declares, argument errors are reported before any launch, and the schedule / mesh /
score-mod helpers agree with the oracle.  No compute call is made here."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

from oracle import oracle as O
from ring_attention_b200 import Mesh, ScoreMod, _lib
from ring_attention_b200._lib import RaScoreMod, RaShape, RaTensor, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        text = open(os.path.join(inc, f)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(ra_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    declared = _header_symbols()
    assert declared, "no declarations found"
    raw = C.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(raw, name), f"{name} is declared in include/ but not exported"
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    assert lib.ra_version() == 1


def _shape(**kw):
    d = dict(b=1, h=1, lq=4, lk=4, dk=8, dv=8, dtype=0, sm_scale=1.0)
    d.update(kw)
    return RaShape(*[d[k] for k in ("b", "h", "lq", "lk", "dk", "dv", "dtype", "sm_scale")])


def _err():
    return lib.ra_last_error_string().decode()


def test_argument_errors_are_negative_and_explained():
    t = RaTensor(0x1000, 1, 1, 1)
    one = C.c_void_p(0x1000)
    args = (C.byref(t), C.byref(t), C.byref(t))
    assert lib.ra_fwd_block(None, *args, None, one, one, one, 1, None) == -1
    rc = lib.ra_fwd_block(C.byref(_shape(lq=0)), *args, None, one, one, one, 1, None)
    assert rc == -2 and "lq" in _err()
    assert lib.ra_fwd_block(C.byref(_shape(dk=512)), *args, None, one, one, one, 1, None) == -3
    assert lib.ra_fwd_block(C.byref(_shape(dtype=7)), *args, None, one, one, one, 1, None) == -4
    assert lib.ra_fwd_block(C.byref(_shape()), None, args[1], args[2], None, one, one, one, 1, None) == -6
    assert lib.ra_fwd_block(C.byref(_shape()), *args, None, None, one, one, 1, None) == -6
    # score-mod combinations ring_self_attention refuses (ring.py:368-374)
    m = RaScoreMod()
    m.kinds = _lib.RA_MOD_CAUSAL | _lib.RA_MOD_PREFIX
    assert lib.ra_fwd_block(C.byref(_shape()), *args, C.byref(m), one, one, one, 1, None) == -8
    m.kinds = _lib.RA_MOD_CAUSAL  # positions missing
    rc = lib.ra_fwd_block(C.byref(_shape()), *args, C.byref(m), one, one, one, 1, None)
    assert rc == -9 and "positions" in _err()
    m.kinds = _lib.RA_MOD_SEGMENT
    assert lib.ra_fwd_block(C.byref(_shape()), *args, C.byref(m), one, one, one, 1, None) == -10
    m.kinds = 1 << 12
    assert lib.ra_fwd_block(C.byref(_shape()), *args, C.byref(m), one, one, one, 1, None) == -7
    assert lib.ra_set_impl(9) == -21
    assert lib.ra_set_impl(_lib.RA_IMPL_AUTO) == 0
    assert lib.ra_ring_source(0, 0, 0) < 0
    assert lib.ra_ring_fwd(None, C.byref(_shape()), *args, None, C.byref(t), one, None) == -30
    # ring plans: handle and result pointer are checked before anything touches a device
    out = C.c_void_p()
    assert lib.ra_ring_plan_create(None, C.byref(_shape()), None, None, C.byref(out)) == -30 and not out.value
    assert lib.ra_ring_use_plan(None, None) == -30
    assert lib.ra_ring_plan_need(None, 0, 0) == -6
    lib.ra_ring_plan_destroy(None)  # like free(NULL)


def test_ring_source_matches_reference_rotation():
    """After t rotations i -> i+1 (ring.py:54) rank r holds the block of rank (r - t) mod N."""
    for n in (1, 2, 3, 4, 8):
        held = list(range(n))
        for t in range(n):
            for r in range(n):
                assert lib.ra_ring_source(r, n, t) == held[r]
            held = [held[(r - 1) % n] for r in range(n)]


def test_mesh_coordinates():
    assert Mesh.coords_of(5, (2, 4)) == (1, 1)
    assert Mesh.axis_ranks(5, 1, (2, 4)) == [4, 5, 6, 7]
    assert Mesh.axis_ranks(5, 0, (2, 4)) == [1, 5]
    assert Mesh.axis_ranks(3, 1, (1, 8)) == list(range(8))  # ring_test.py:60-65


@pytest.mark.parametrize("causal,seg,prefix,alibi,window", [
    (True, False, False, False, 0), (True, True, False, False, 0), (False, True, False, False, 0),
    (False, True, True, False, 0), (True, False, False, True, 7), (False, False, False, False, 5),
])
def test_score_mod_dense_form_matches_oracle(causal, seg, prefix, alibi, window):
    rng = np.random.default_rng(0)
    b, h, lq, lk = 2, 3, 20, 28
    qpos = rng.integers(0, 40, (b, lq)).astype(np.int32)
    kpos = rng.integers(0, 40, (b, lk)).astype(np.int32)
    qseg = rng.integers(0, 3, (b, lq)).astype(np.int32) if seg else None
    kseg = rng.integers(0, 3, (b, lk)).astype(np.int32) if seg else None
    qpre = rng.integers(0, 2, (b, lq)).astype(bool) if prefix else None
    kpre = rng.integers(0, 2, (b, lk)).astype(bool) if prefix else None
    slopes = O.alibi_slopes(h) if alibi else None
    want = O.score_mod_bias(b, h, qpos, kpos, qseg, kseg, qpre, kpre, causal, slopes, window)
    T = lambda a: None if a is None else torch.from_numpy(a)
    mod = ScoreMod(causal=causal, alibi_slopes=T(slopes), window=window)
    got = mod(q_segment_ids=T(qseg), kv_segment_ids=T(kseg), q_positions=T(qpos), kv_positions=T(kpos),
              q_prefix_mask=T(qpre), kv_prefix_mask=T(kpre)).numpy()
    np.testing.assert_allclose(np.broadcast_to(got, want.shape), want, rtol=1e-6)
    kinds = mod.kinds({"q_segment_ids": qseg, "q_prefix_mask": qpre}, {})
    assert bool(kinds & _lib.RA_MOD_CAUSAL) == causal
    assert bool(kinds & _lib.RA_MOD_SEGMENT) == seg
    assert bool(kinds & _lib.RA_MOD_PREFIX) == (prefix and not causal)


def test_api_refuses_cpu_tensors_and_unknown_impl():
    import ring_attention_b200 as ra

    q = torch.zeros(1, 4, 1, 8)
    with pytest.raises(ValueError):
        ra.ring_attention(q, q, q, "sp", block_impl="numpy")  # ring.py:311-312
    with pytest.raises(ra.RingAttentionError):
        ra.ring_attention(q, q, q, "sp")
    with pytest.raises(AssertionError):
        ra.ring_self_attention(q, q, q, None, ("dp", "sp", None), causal=True)  # ring.py:368-370


def test_zigzag_layout_round_trip_and_balance():
    import ring_attention_b200 as ra

    n, S = 4, 64
    x = torch.arange(2 * S * 3).reshape(2, S, 3)
    shards = [ra.zigzag_shard(x, r, n) for r in range(n)]
    assert all(s.shape == (2, S // n, 3) for s in shards)
    assert torch.equal(ra.zigzag_unshard(shards), x)
    # every rank sees the same number of causal (query, key) pairs at every step
    pos = [ra.zigzag_indices(S, r, n) for r in range(n)]
    for t in range(n):
        counts = []
        for r in range(n):
            src = lib.ra_ring_source(r, n, t)
            counts.append(int((pos[src][None, :] <= pos[r][:, None]).sum()))
        assert max(counts) - min(counts) <= S // n, counts
    with pytest.raises(ValueError):
        ra.zigzag_indices(30, 0, 4)


def test_bench_workload_pair_counts():
    """bench.py counts visible (query, key) pairs exactly; check each mask's closed form against a
    brute-force count on a small sequence."""
    import bench

    s = 1536
    i, j = np.arange(s)[:, None], np.arange(s)[None, :]
    w = dict(b=1, h=1, d=64, s=s, mask="causal")
    assert bench.visible_pairs(w) == int((j <= i).sum())
    w = dict(b=1, h=1, d=64, s=s, mask="alibi+window", window=200)
    assert bench.visible_pairs(w) == int(((j <= i) & (i - j < 200)).sum())
    w = dict(b=1, h=1, d=64, s=40000, mask="documents")
    lens = bench.document_lengths(40000)
    assert sum(lens) == 40000 and all(512 <= n <= 16384 for n in lens[:-1]) and 1 <= lens[-1] <= 16384
    seg = np.repeat(np.arange(len(lens)), lens)
    brute = sum(int(n) * (int(n) + 1) // 2 for n in np.bincount(seg))
    assert bench.visible_pairs(w) == brute
    # forward-only workloads count 4d FLOP per pair, the others 14d
    assert bench.flops(dict(w, backward=False)) * 14 == bench.flops(w) * 4
    assert bench.metric_name(dict(backward=False)).endswith("fwd_tokens_per_s")


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: it times the oracle port on the host cores and
    prints one JSON line with the keys the benchmark contract names."""
    import json
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["value"] > 0 and line["unit"] == "tokens/s"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and "workload" in line["config"]
