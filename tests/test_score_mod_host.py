"""The score-mod rules of the kernels, compiled for the host and checked without a GPU.

`csrc/score_mod.h` holds the per-pair visibility rule (`apply_mod`) and the rule that decides,
from the 128-token summaries of a query tile and a key tile, whether the kernels skip the tile
pair (every pair masked), run it without mask arithmetic (every pair visible) or take the
masking pass (`classify_tiles`; the ring plan uses the same rule to leave out ring steps and
rows of K/V blocks).  A wrong "skip" or "all visible" silently drops or adds attention mass, so:

* `apply_mod` is compared with a NumPy restatement of the reference's mask builder
  (ring.py:386-408) plus the window and ALiBi terms;
* for thousands of random tile pairs (contiguous, strided, shuffled and constant positions;
  one or several documents per tile; every kind of prefix flags) and all 16 combinations of
  mask kinds, "skip" must mean no visible pair and "all visible" must mean 128 x 128 of them,
  counted with `apply_mod` itself;
* on tiles of contiguous positions that lie in one document each, the classification must be
  exact for causal, window and document masks: that is what the skipped work at long sequence
  lengths rests on.

The shim is built with g++ from the same header the CUDA sources include.
"""
import ctypes
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CAUSAL, SEGMENT, PREFIX, ALIBI, WINDOW = 1, 2, 4, 8, 16
T = 128


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("shim") / "score_mod_shim.so")
    cmd = ["g++", "-O1", "-shared", "-fPIC", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I",
           os.path.join(ROOT, "ring_attention_b200", "csrc"), os.path.join(ROOT, "tests", "host_shim", "score_mod_shim.cpp"),
           "-o", out]
    subprocess.run(cmd, check=True, capture_output=True)
    lib = ctypes.CDLL(out)
    i32p, u8p = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_uint8)
    lib.ra_host_classify.argtypes = [ctypes.c_uint32, ctypes.c_int32, i32p, i32p]
    lib.ra_host_classify.restype = ctypes.c_int
    lib.ra_host_count_visible.argtypes = [ctypes.c_uint32, ctypes.c_int32, ctypes.c_int, i32p, i32p, u8p, ctypes.c_int,
                                          i32p, i32p, u8p]
    lib.ra_host_count_visible.restype = ctypes.c_int64
    lib.ra_host_apply_mod.argtypes = [ctypes.c_float, ctypes.c_uint32, ctypes.c_int32, ctypes.c_float] + \
        [ctypes.c_int32, ctypes.c_int32, ctypes.c_int] * 2 + [ctypes.POINTER(ctypes.c_float)]
    lib.ra_host_apply_mod.restype = ctypes.c_int
    return lib


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


def meta(pos, seg, pre):
    contig = int(np.array_equal(pos, pos[0] + np.arange(len(pos))))
    return np.array([pos.min(), pos.max(), seg.min(), seg.max(), int(pre.any()), int(pre.all()), contig], np.int32)


def classify(lib, kinds, window, q, k):
    return lib.ra_host_classify(kinds, window, _p(meta(*q), ctypes.c_int32), _p(meta(*k), ctypes.c_int32))


def count_visible(lib, kinds, window, q, k):
    return lib.ra_host_count_visible(kinds, window, T, _p(q[0], ctypes.c_int32), _p(q[1], ctypes.c_int32),
                                     _p(q[2], ctypes.c_uint8), T, _p(k[0], ctypes.c_int32), _p(k[1], ctypes.c_int32),
                                     _p(k[2], ctypes.c_uint8))


def random_tile(rng, base):
    kind = rng.integers(0, 5)
    if kind == 0:
        pos = base + np.arange(T)
    elif kind == 1:
        pos = base + np.sort(rng.choice(4 * T, T, replace=False))
    elif kind == 2:
        pos = base + rng.permutation(T)
    elif kind == 3:
        pos = base + rng.integers(0, 3 * T, T)
    else:
        pos = np.full(T, base)
    sk = rng.integers(0, 4)
    if sk == 0:
        seg = np.full(T, rng.integers(0, 3))
    elif sk == 1:
        seg = np.sort(rng.integers(0, 3, T)) + rng.integers(0, 2)
    elif sk == 2:
        seg = rng.integers(0, 4, T)
    else:
        cut = rng.integers(1, T)
        s0 = rng.integers(0, 3)
        seg = np.where(np.arange(T) < cut, s0, s0 + 1)
    pk = rng.integers(0, 4)
    pre = [np.zeros(T), np.ones(T), rng.integers(0, 2, T), np.arange(T) < rng.integers(0, T + 1)][pk]
    return pos.astype(np.int32), seg.astype(np.int32), pre.astype(np.uint8)


def numpy_visible(kinds, window, q, k):
    """ring.py:386-408 (segments, causal or prefix-LM) plus the sliding window."""
    qp, qs, qr = (a[:, None].astype(np.int64) for a in q)
    kp, ks, kr = (a[None, :].astype(np.int64) for a in k)
    vis = np.ones((len(q[0]), len(k[0])), bool)
    if kinds & SEGMENT:
        vis &= qs == ks
    if kinds & CAUSAL:
        vis &= kp <= qp
    elif kinds & PREFIX:
        vis &= ((qr != 0) & (kr != 0)) | (kp <= qp)
    if kinds & WINDOW:
        vis &= (qp - kp) < window
    return vis


def test_apply_mod_is_the_reference_mask_rule(shim):
    rng = np.random.default_rng(0)
    out = ctypes.c_float()
    for _ in range(4000):
        kinds = int(rng.integers(0, 32))
        window = int(rng.choice([1, 3, 64, 4096]))
        qpos, kpos = int(rng.integers(-5, 300)), int(rng.integers(-5, 300))
        qseg, kseg = int(rng.integers(0, 3)), int(rng.integers(0, 3))
        qpre, kpre = int(rng.integers(0, 2)), int(rng.integers(0, 2))
        slope, s = float(rng.random()), float(rng.normal())
        vis = shim.ra_host_apply_mod(s, kinds, window, slope, qpos, qseg, qpre, kpos, kseg, kpre, ctypes.byref(out))
        q = (np.array([qpos]), np.array([qseg]), np.array([qpre]))
        k = (np.array([kpos]), np.array([kseg]), np.array([kpre]))
        want = bool(numpy_visible(kinds, window, q, k)[0, 0])
        assert bool(vis) == want, (kinds, window, qpos, kpos, qseg, kseg, qpre, kpre)
        if want:
            bias = -np.float32(slope) * np.float32(qpos - kpos) if kinds & ALIBI else np.float32(0)
            assert out.value == np.float32(np.float32(s) + bias)
        else:
            assert out.value == -np.inf


def test_classification_never_promises_too_much(shim):
    rng = np.random.default_rng(1)
    seen = {0: 0, 1: 0, 2: 0}
    for _ in range(1500):
        qbase = int(rng.integers(0, 6 * T))
        kbase = qbase + int(rng.choice([-5 * T, -2 * T, -T, -T // 2, 0, 1, T // 2, T, 2 * T]))
        q, k = random_tile(rng, qbase), random_tile(rng, kbase)
        for kinds in range(0, 32):
            if kinds & ALIBI:
                continue
            window = int(rng.choice([1, 17, T, 200, 4 * T]))
            cls = classify(shim, kinds, window, q, k)
            seen[cls] += 1
            if cls == 2:
                continue
            n = count_visible(shim, kinds, window, q, k)
            assert n == (0 if cls == 0 else T * T), (kinds, window, cls, n, meta(*q), meta(*k))
            assert n == int(numpy_visible(kinds, window, q, k).sum())
    assert min(seen.values()) > 500, seen  # every answer was exercised


@pytest.mark.parametrize("kinds", [CAUSAL, CAUSAL | WINDOW, CAUSAL | SEGMENT, CAUSAL | SEGMENT | WINDOW, WINDOW, SEGMENT])
def test_classification_is_exact_on_contiguous_single_document_tiles(shim, kinds):
    rng = np.random.default_rng(2)
    zeros = np.zeros(T, np.uint8)
    for _ in range(600):
        window = int(rng.choice([T, 2 * T, 3 * T + 5, 4096]))
        qt, kt = int(rng.integers(0, 40)), int(rng.integers(0, 40))
        q = ((qt * T + np.arange(T)).astype(np.int32), np.full(T, rng.integers(0, 2), np.int32), zeros)
        k = ((kt * T + np.arange(T)).astype(np.int32), np.full(T, rng.integers(0, 2), np.int32), zeros)
        n = int(numpy_visible(kinds, window, q, k).sum())
        want = 0 if n == 0 else (1 if n == T * T else 2)
        assert classify(shim, kinds, window, q, k) == want, (kinds, window, qt, kt, n)
