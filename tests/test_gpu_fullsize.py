"""Parity at the benchmark configurations' sizes, by sampled rows.

A dense float64 oracle over 32k-128k tokens is out of reach, so for a sample of query rows
the oracle attends that row to all keys (O(S d) per row) and out, L and dQ of those rows are
compared; dK/dV are compared on a sample of key rows using the oracle's own L for every query
of one (batch, head), computed blockwise.  Masks are built by the same generators as the
small-size tests (causal, packed documents, ALiBi + sliding window).
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import BF16_ATOL, BF16_RTOL, round_bf16, to_dev

pytestmark = pytest.mark.gpu


def ra():
    import ring_attention_b200

    return ring_attention_b200


def _close(got, want, what):
    err = np.abs(got - want)
    bound = BF16_ATOL + BF16_RTOL * np.abs(want)
    assert np.all(err <= bound), f"{what}: max err {err.max():.3e}, worst excess {(err - bound).max():.3e}"


def _row_oracle(q, k, v, do, rows, vis_fn, slopes, scale, hh):
    """out, L, dq of the sampled query rows of head hh ([S, d] arrays, float64)."""
    outs, Ls, dqs = [], [], []
    for i in rows:
        s = (k @ q[i]) * scale
        vis, rel = vis_fn(i)
        if slopes is not None:
            s = s - slopes[hh] * rel
        s = np.where(vis, s, -np.inf)
        m = s.max()
        p = np.exp(s - m)
        l = p.sum()
        a = p / l
        o = a @ v
        dp = v @ do[i]
        ds = a * (dp - do[i] @ o) * scale
        outs.append(o)
        Ls.append(m + np.log(l))
        dqs.append(ds @ k)
    return np.array(outs), np.array(Ls), np.array(dqs)


CASES = [
    # name, b, h, S, d, kind, backward
    ("causal_32k", 1, 2, 32768, 128, "causal", True),
    ("documents_64k", 1, 2, 65536, 128, "documents", True),
    ("alibi_window_32k_d64", 1, 4, 32768, 64, "alibi+window", False),
]


@pytest.mark.parametrize("name,b,h,S,d,kind,backward", CASES, ids=[c[0] for c in CASES])
def test_sampled_rows_at_benchmark_sizes(name, b, h, S, d, kind, backward):
    rng = np.random.default_rng(42)
    q, k, v, do = (round_bf16(rng.standard_normal((b, S, h, d))) for _ in range(4))
    pos = np.broadcast_to(np.arange(S, dtype=np.int32), (b, S)).copy()
    seg, slopes, window = None, None, 0
    if kind == "documents":
        seg1, _ = O.pack_documents(S, 512, 16384, seed=0)
        seg = np.broadcast_to(seg1, (b, S)).copy()
    if kind == "alibi+window":
        slopes, window = O.alibi_slopes(h), 4096
    scale = 1 / np.sqrt(d)

    def vis_fn(i):
        rel = (i - np.arange(S)).astype(np.float64)
        vis = rel >= 0
        if seg is not None:
            vis &= seg[0] == seg[0, i]
        if window:
            vis &= rel < window
        return vis, rel

    T = lambda a, t=torch.int32: None if a is None else to_dev(a, t)
    sm = ra().ScoreMod(causal=True, alibi_slopes=T(slopes, torch.float32), window=window)
    qkw = {"q_positions": T(pos), "q_segment_ids": T(seg)}
    kkw = {"kv_positions": T(pos), "kv_segment_ids": T(seg)}
    tq, tk, tv, tdo = (to_dev(x, torch.bfloat16) for x in (q, k, v, do))
    tq.requires_grad_(True), tk.requires_grad_(True), tv.requires_grad_(True)
    out = ra().ring_attention(tq, tk, tv, "sp", bias_fn=sm, bias_q_kwargs=qkw, bias_kv_kwargs=kkw, block_impl="tcgen05")
    if backward:
        out.backward(tdo)
    torch.cuda.synchronize()
    rows = np.unique(np.concatenate([[0, 1, 127, 128, S - 1], rng.integers(0, S, 40)]))
    hh = h - 1
    ro, rL, rdq = _row_oracle(q[0, :, hh], k[0, :, hh], v[0, :, hh], do[0, :, hh], rows, vis_fn, slopes, scale, hh)
    _close(out.detach()[0, rows, hh].float().cpu().numpy().astype(np.float64), ro, "out")
    if backward:
        _close(tq.grad[0, rows, hh].float().cpu().numpy().astype(np.float64), rdq, "dq")
        # dK/dV of sampled key rows: needs L and delta of every query of this head (blockwise oracle)
        kq, kk_, kv_, kdo = q[0, :, hh], k[0, :, hh], v[0, :, hh], do[0, :, hh]
        cols = np.unique(np.concatenate([[0, 127, S - 1], rng.integers(0, S, 12)]))
        L = np.empty(S)
        delta = np.empty(S)
        blk = 2048
        for s0 in range(0, S, blk):
            e0 = min(s0 + blk, S)  # causal: keys beyond the block's last row are never visible
            sc = (kq[s0:e0] @ kk_[:e0].T) * scale
            vis = np.arange(s0, e0)[:, None] >= np.arange(e0)[None, :]
            if seg is not None:
                vis &= seg[0, s0:e0, None] == seg[0, None, :e0]
            sc[~vis] = -np.inf
            m = sc.max(-1)
            p = np.exp(sc - m[:, None])
            l = p.sum(-1)
            L[s0:e0] = m + np.log(l)
            delta[s0:e0] = np.einsum("id,id->i", (p / l[:, None]) @ kv_[:e0], kdo[s0:e0])
        for j in cols:
            sj = (kq @ kk_[j]) * scale
            visj = np.array([True] * S)
            relj = np.arange(S) - j
            visj &= relj >= 0
            if seg is not None:
                visj &= seg[0] == seg[0, j]
            pj = np.where(visj, np.exp(sj - L), 0.0)
            dv_j = pj @ kdo
            ds_j = pj * (kdo @ kv_[j] - delta) * scale
            dk_j = ds_j @ kq
            _close(tk.grad[0, j, hh].float().cpu().numpy().astype(np.float64), dk_j, f"dk[{j}]")
            _close(tv.grad[0, j, hh].float().cpu().numpy().astype(np.float64), dv_j, f"dv[{j}]")
