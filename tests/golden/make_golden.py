"""Writes tests/golden/*.npz: outputs of the REFERENCE's own code on seeded inputs.

The reference project stores no golden arrays, and JAX cannot be installed here.  Its ring.py
is therefore run on a NumPy stand-in for the JAX names it uses (jax_on_numpy.py, reference_run.py:
one thread per virtual device, float64); what executes is the reference's Python: the public
entry points, the custom-VJP forward and backward scans, the block functions, the rotation and
the mask builder (`block_impl="jax"`; tests/test_reference_run.py also runs the Pallas kernels).  The fixtures hold those
outputs in float32 and travel to machines without the reference checkout.  Where the checkout is
absent this script falls back to the CPU oracle (`source` in each file says which it was).
Inputs are not stored; `inputs(case)` below regenerates them from a seeded NumPy PCG64
stream.  Run from the repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402

# name -> (seed, b, q_len, kv_len, h, d, nranks, mask)
# shapes: ring_test.py:49-52 (forward), :105-110 (backward), :323-328 (self attention),
# and the CPU-runnable benchmark configuration (b1 h4 S1024 d64, 4 ranks, causal).
CASES = {
    "tiny_cross": (0, 2, 24, 16, 1, 2, 8, "none"),
    "cross_128_64": (1, 2, 128, 64, 4, 64, 8, "none"),
    "cross_64_512": (2, 2, 64, 512, 4, 16, 8, "none"),
    "segments_128_64": (1, 2, 128, 64, 4, 64, 8, "segments"),
    "self_causal_seg_512": (2, 2, 512, 512, 4, 16, 8, "causal+segments"),
    "config1_causal_1024": (0, 1, 1024, 1024, 4, 64, 4, "causal"),
    "self_prefix_seg_256": (4, 2, 256, 256, 2, 32, 8, "prefix+segments"),
}


def inputs(name):
    seed, b, lq, lk, h, d, n, mask = CASES[name]
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((b, lq, h, d)).astype(np.float32)
    k = rng.standard_normal((b, lk, h, d)).astype(np.float32)
    v = rng.standard_normal((b, lk, h, d)).astype(np.float32)
    do = rng.standard_normal((b, lq, h, d)).astype(np.float32)
    extra = {}
    if mask == "segments":  # ring_test.py:203-208: independent ids in [0, q_len // 5)
        extra["q_seg"] = rng.integers(0, lq // 5, (b, lq)).astype(np.int32)
        extra["kv_seg"] = rng.integers(0, lq // 5, (b, lk)).astype(np.int32)
    if mask == "causal+segments":  # ring_test.py:347-350
        extra["q_seg"] = extra["kv_seg"] = rng.integers(0, 5, (b, lq)).astype(np.int32)
    if mask == "prefix+segments":  # ring.py:399-406: bidirectional inside the prefix, causal after it
        extra["q_seg"] = extra["kv_seg"] = np.sort(rng.integers(0, 3, (b, lq)), axis=1).astype(np.int32)
        extra["q_pre"] = extra["kv_pre"] = np.arange(lq)[None] % 97 < rng.integers(8, 60, (b, 1))
    if "causal" in mask or "prefix" in mask:
        extra["q_pos"] = np.broadcast_to(np.arange(lq, dtype=np.int32), (b, lq)).copy()
        extra["kv_pos"] = np.broadcast_to(np.arange(lk, dtype=np.int32), (b, lk)).copy()
    return q, k, v, do, extra


def dense_bias(name, extra):
    seed, b, lq, lk, h, d, n, mask = CASES[name]
    if mask == "none":
        return None
    return O.score_mod_bias(b, h, q_positions=extra.get("q_pos"), kv_positions=extra.get("kv_pos"),
                            q_segment_ids=extra.get("q_seg"), kv_segment_ids=extra.get("kv_seg"),
                            q_prefix_mask=extra.get("q_pre"), kv_prefix_mask=extra.get("kv_pre"),
                            causal="causal" in mask)


def answers(name):
    q, k, v, do, extra = inputs(name)
    bias = dense_bias(name, extra)
    out, lse = O.mha(q, k, v, bias, return_lse=True)
    dq, dk, dv = O.mha_grads(q, k, v, do, bias)
    return {"out": out, "lse": lse, "dq": dq, "dk": dk, "dv": dv}


def reference_answers(name):
    """The same five arrays from the reference's own code (reference_run.py)."""
    sys.path.insert(0, HERE)
    import reference_run as R

    seed, b, lq, lk, h, d, n, mask = CASES[name]
    q, k, v, do, extra = inputs(name)
    if mask in ("none", "segments"):  # the general entry point; independent ids for queries and keys
        return R.reference_answers(q, k, v, do, n, q_seg=extra.get("q_seg"), kv_seg=extra.get("kv_seg"))
    return R.reference_answers(q, k, v, do, n, q_seg=extra.get("q_seg"), kv_seg=extra.get("kv_seg"),
                               q_pos=extra.get("q_pos"), kv_pos=extra.get("kv_pos"), q_pre=extra.get("q_pre"),
                               kv_pre=extra.get("kv_pre"), causal="causal" in mask, api="ring_self_attention")


def main():
    sys.path.insert(0, HERE)
    import reference_run as R

    from_reference = R.available()
    for name in CASES:
        ans = reference_answers(name) if from_reference else answers(name)
        ans["source"] = np.array("reference ring.py on the NumPy stand-in" if from_reference else "oracle")
        source = ans.pop("source")
        if name.startswith("config1"):  # keep the file small: every 16th row
            ans = {k2: (a[:, ::16] if k2 != "lse" else a[:, :, ::16]) for k2, a in ans.items()}
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, source=source, **{k2: a.astype(np.float32) for k2, a in ans.items()})
        print(path, os.path.getsize(path))


if __name__ == "__main__":
    main()
