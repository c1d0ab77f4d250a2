"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import oracle as O

F32_ATOL = 1e-5            # max-abs bound for float32 results against the float64 oracle
BF16_ATOL, BF16_RTOL = 2e-2, 1e-2  # bf16 results against the oracle run on the bf16-rounded inputs


def to_dev(x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to("cuda", dtype)


def round_bf16(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16).to(torch.float64).numpy()


def check_close(got, want, dtype, what="", f32_atol=F32_ATOL, nan="match"):
    """nan="match": NaNs must sit exactly where the oracle has them.  nan="finite": where the
    oracle is NaN (gradients poisoned by a row that saw no key, ring.py:146) the engine's
    compiled-in masks give finite values instead; those entries are only checked for that."""
    got = got.detach().to(torch.float64).cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    if nan == "match":
        np.testing.assert_array_equal(np.isnan(got), np.isnan(want), err_msg=f"{what}: NaN pattern")
    else:
        assert not np.isnan(got).any(), f"{what}: unexpected NaN"
    np.testing.assert_array_equal(np.isneginf(got), np.isneginf(want), err_msg=f"{what}: -inf pattern")
    ok = np.isfinite(want)
    err = np.abs(got[ok] - want[ok])
    if dtype == torch.float32:
        assert err.size == 0 or err.max() <= f32_atol, f"{what}: max abs err {err.max():.3e} > {f32_atol}"
    else:
        bound = BF16_ATOL + BF16_RTOL * np.abs(want[ok])
        assert np.all(err <= bound), f"{what}: max abs err {err.max():.3e}, worst excess {(err - bound).max():.3e}"


def make_inputs(seed, b, lq, lk, h, d, dtype, dv=None, std=1.0):
    rng = np.random.default_rng(seed)
    dv = dv or d
    q = rng.standard_normal((b, lq, h, d)) * std
    k = rng.standard_normal((b, lk, h, d)) * std
    v = rng.standard_normal((b, lk, h, dv)) * std
    do = rng.standard_normal((b, lq, h, dv))
    if dtype == torch.bfloat16:
        q, k, v, do = (round_bf16(x) for x in (q, k, v, do))
    else:
        q, k, v, do = (x.astype(np.float32).astype(np.float64) for x in (q, k, v, do))
    return q, k, v, do, rng
