"""Parity at the benchmark configurations' own sizes, by sampled rows.

A dense float64 oracle over 32k-128k tokens is out of reach, so for a sample of query rows
the oracle attends that row to all keys (O(S d) per row) and out, L and dQ of those rows are
compared; dK/dV are compared on a sample of key rows, for which the oracle computes L and
delta of every query that sees them (`oracle.sampled_rows`).  Inputs are drawn on the device
from a seeded generator (the host only ever holds the one (batch, head) slice it checks);
masks are built by the same generators as the small-size tests (causal, packed documents,
ALiBi + sliding window).  Everything runs through the C ABI (`ra_ring_fwd` / `ra_ring_bwd`
on a ring of one).
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import BF16_ATOL, BF16_RTOL

pytestmark = pytest.mark.gpu


def ra():
    import ring_attention_b200

    return ring_attention_b200


def _close(got, want, what):
    got = got.detach().to(torch.float64).cpu().numpy()
    np.testing.assert_array_equal(np.isfinite(got), np.isfinite(want), err_msg=f"{what}: finite pattern")
    err = np.abs(got - want)
    bound = BF16_ATOL + BF16_RTOL * np.abs(want)
    assert np.all(err <= bound), f"{what}: max err {err.max():.3e}, worst excess {(err - bound).max():.3e}"


CASES = [
    # name, b, h, S, d, kind, backward, std, which key rows get dK/dV checked
    ("causal_32k", 1, 2, 32768, 128, "causal", True, 1.0, "any"),
    # BASELINE config 3: the real document packing over the full 131072 tokens, a head subset
    ("documents_128k", 1, 2, 131072, 128, "documents", True, 1.0, "any"),
    # BASELINE config 4 at its own shape
    ("alibi_window_64k_d64", 4, 16, 65536, 64, "alibi+window", False, 1.0, "none"),
    # BASELINE config 5: one 131072 x 131072 block (what one GPU holds), N(0, 0.5^2) inputs; dK/dV
    # rows only among the last 1024 positions (a key row early in the sequence is seen by ~all queries)
    ("causal_128k_block", 1, 2, 131072, 128, "causal", True, 0.5, "late"),
]


@pytest.mark.parametrize("name,b,h,S,d,kind,backward,std,krows", CASES, ids=[c[0] for c in CASES])
def test_sampled_rows_at_benchmark_sizes(name, b, h, S, d, kind, backward, std, krows):
    from ring_attention_b200 import ring as R

    g = torch.Generator(device="cuda").manual_seed(42)
    q, k, v, do = ((torch.randn((b, S, h, d), generator=g, device="cuda") * std).to(torch.bfloat16) for _ in range(4))
    rng = np.random.default_rng(42)
    pos = torch.arange(S, dtype=torch.int32, device="cuda").expand(b, S).contiguous()
    seg1, slopes, window = None, None, 0
    if kind == "documents":
        seg1, _ = O.pack_documents(S, 512, 16384, seed=0)
    if kind == "alibi+window":
        slopes, window = O.alibi_slopes(h), 4096
    scale = 1 / np.sqrt(d)
    seg = None if seg1 is None else torch.from_numpy(seg1).to("cuda", torch.int32).expand(b, S).contiguous()
    sm = ra().ScoreMod(causal=True, window=window,
                       alibi_slopes=None if slopes is None else torch.from_numpy(slopes).to("cuda", torch.float32))
    qkw = {"q_positions": pos, "q_segment_ids": seg}
    kkw = {"kv_positions": pos, "kv_segment_ids": seg}
    ring = ra().mesh.resolve_axis("sp")
    from ring_attention_b200 import _lib

    assert _lib.lib.ra_set_impl(_lib.RA_IMPL_TCGEN05) == 0
    out, lse = R._fused_fwd(ring, q, k, v, scale, sm, qkw, kkw)
    if backward:
        dq, dk, dv = R._fused_bwd(ring, q, k, v, out, lse, do, scale, sm, qkw, kkw)
    assert _lib.lib.ra_set_impl(_lib.RA_IMPL_AUTO) == 0
    assert ra().device_status() == 0

    bb, hh = b - 1, h - 1
    f = lambda t: t[bb, :, hh].to(torch.float64).cpu().numpy()
    rows = np.unique(np.concatenate([[0, 1, 127, 128, S - 1], rng.integers(0, S, 40)]))
    if krows == "any":
        cols = np.unique(np.concatenate([[0, 127, S - 1], rng.integers(0, S, 5)]))
    elif krows == "late":
        cols = np.unique(np.concatenate([[S - 1, S - 128, S - 129], rng.integers(S - 1024, S, 5)]))
    else:
        cols = np.array([], np.int64)
    want = O.sampled_rows(f(q), f(k), f(v), f(do), scale, rows, cols if backward else [], seg=seg1, window=window,
                          slope=None if slopes is None else slopes[hh], causal=True, score_dtype=np.float32)
    _close(out[bb, rows, hh], want["out"], "out")
    # L = m + log(l) of ring.py:135: compared like every other result
    _close(lse[bb, hh, rows], want["L"], "L")
    if backward:
        _close(dq[bb, rows, hh], want["dq"], "dq")
        _close(dk[bb, cols, hh], want["dk"], "dk")
        _close(dv[bb, cols, hh], want["dv"], "dv")
