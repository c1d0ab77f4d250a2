"""bench.py's own parity check (sampled rows against the oracle, every rank, every N) on CPU:
results computed by the dense oracle must pass, for both token layouts, and a result that is
wrong in one sampled place must fail.  Guards the index bookkeeping (shards rebuilt from
seeds, zig-zag positions, local <-> global rows) that the GPU runs rely on."""
import types

import numpy as np
import pytest
import torch

import bench
from oracle import oracle as O


def _dense_results(w, layout, N, seg_global, slopes):
    b, h, d, S = w["b"], w["h"], w["d"], w["s"]
    c = S // N
    full = [np.zeros((b, S, h, d)) for _ in range(4)]
    idxs = [bench.shard_indices(layout, S, r, N).numpy() for r in range(N)]
    for r in range(N):
        for t in range(4):
            for hd in range(h):
                full[t][:, idxs[r], hd] = bench.shard_slice(r, t, hd, b, c, d, 1.0, torch.bfloat16).double().numpy()
    pos = np.broadcast_to(np.arange(S), (b, S))
    sg = None if seg_global is None else np.broadcast_to(seg_global, (b, S))
    bias = O.score_mod_bias(b, h, pos, pos, sg, sg, causal=True, window=w.get("window", 0), alibi_slopes=slopes)
    out, L = O.mha(*full[:3], bias, return_lse=True)
    dq, dk, dv = O.mha_grads(*full, bias)
    per_rank = []
    for r in range(N):
        i = idxs[r]
        T = torch.from_numpy
        per_rank.append({"out": T(out[:, i]), "lse": T(L[:, :, i]), "dq": T(dq[:, i]), "dk": T(dk[:, i]), "dv": T(dv[:, i])})
    return per_rank


@pytest.mark.parametrize("layout,N,mask", [("zigzag", 4, "causal"), ("contiguous", 2, "documents"), ("zigzag", 1, "causal")])
def test_parity_check_accepts_oracle_results_and_rejects_a_wrong_row(layout, N, mask):
    w = dict(dtype="bf16", b=2, h=3, d=16, s=512, mask=mask)
    args = types.SimpleNamespace(layout=layout)
    seg = None
    if mask == "documents":
        seg, _ = O.pack_documents(512, 20, 120, seed=0)
    res = _dense_results(w, layout, N, seg, None)
    for r in range(N):
        v = bench.parity_check(w, args, r, N, res[r], seg, None, True)
        assert v["ok"] and v["rows"] >= 2 and v["key_rows"] >= 1, v
        assert v["max_excess"] <= 0
    # one wrong value in a sampled query row of rank N-1
    r = N - 1
    bad = {k: t.clone() for k, t in res[r].items()}
    hh = (r * 5 + 3) % w["h"]
    bad["out"][w["b"] - 1, 0, hh, 0] += 1.0  # local row 0 is always sampled
    assert not bench.parity_check(w, args, r, N, bad, seg, None, True)["ok"]
    bad = {k: t.clone() for k, t in res[r].items()}
    bad["lse"][w["b"] - 1, hh, :] += 0.5
    assert not bench.parity_check(w, args, r, N, bad, seg, None, True)["ok"]


def test_forward_only_workload_checks_out_and_L_only():
    w = dict(dtype="bf16", b=1, h=2, d=16, s=256, mask="alibi+window", window=64, backward=False)
    args = types.SimpleNamespace(layout="contiguous")
    slopes = O.alibi_slopes(2)
    res = _dense_results(w, "contiguous", 2, None, slopes)
    v = bench.parity_check(w, args, 1, 2, res[1], None, slopes, False)
    assert v["ok"] and v["key_rows"] == 0 and set(v["excess"]) == {"out", "L"}
