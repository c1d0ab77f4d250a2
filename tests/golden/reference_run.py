"""Runs the reference's own ring attention (ring_attention/ring.py, `block_impl="jax"`) on the
NumPy stand-in of jax_on_numpy.py, with one thread per virtual device, in float64.

`reference_answers(...)` returns out, L and the gradients of sum(out * do) for one case, computed
by the reference's functions themselves: `ring_attention` / `ring_self_attention`, the custom-VJP
pair `_ring_attention_fwd` / `_ring_attention_bwd`, `_fwd_block` / `_bwd_block`, `_rotate_block`
and the built-in mask builder; with `block_impl="pallas"` also the kernels of ring_kernel.py,
through the stand-in's interpreter of the Pallas calls they make.  Needs the reference checkout:
the directory named by the environment variable REFERENCE_DIR, else a checkout called
`reference` beside this repository; without either the callers skip.  Nothing here ships with
the product.
"""
from __future__ import annotations

import importlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import jax_on_numpy as standin  # noqa: E402

REFERENCE_DIR = os.environ.get("REFERENCE_DIR") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")


def available() -> bool:
    return os.path.exists(os.path.join(REFERENCE_DIR, "ring_attention", "ring.py"))


def load_reference():
    """Imports the reference's ring module from where it lies, on the stand-in."""
    standin.install()
    if REFERENCE_DIR not in sys.path:
        sys.path.insert(0, REFERENCE_DIR)
    return importlib.import_module("ring_attention.ring")


def reference_answers(q, k, v, do, nranks, *, q_seg=None, kv_seg=None, q_pos=None, kv_pos=None,
                      q_pre=None, kv_pre=None, causal=False, api="ring_attention", block_impl="jax",
                      dtype=np.float64):
    """q [b, lq, h, dk], k, v [b, lk, h, d], do like out; integer / bool arrays [b, l].

    api="ring_attention": the general entry point with a segment-id `bias_fn` written like the
    reference's own test helper (a pair is visible when the ids are equal); cross attention allowed.
    api="ring_self_attention": the full-service entry point with its built-in mask (segments,
    causal by positions, prefix-LM); q, k, v must have one length.
    block_impl="pallas" runs the kernels of ring_kernel.py through the stand-in's Pallas
    interpreter (tiles of min(length, 128) rows, ring.py:299-308); they carry m and l in float32.
    """
    ref = load_reference()
    jnp = sys.modules["jax.numpy"]
    q, k, v, do = (np.asarray(x, dtype=dtype) for x in (q, k, v, do))
    spec = standin.PartitionSpec(None, "sp")
    mesh = standin.Mesh(nranks)

    def tail(do_shard):
        res = standin.residuals_of_last_call()
        dq, dk, dv = standin.vjp_of_last_call(do_shard)[:3]
        return np.transpose(np.asarray(res[4]), (0, 2, 1)), dq, dk, dv  # L as [b, l, h]

    if api == "ring_attention":
        bias_fn = None
        if q_seg is not None:
            def bias_fn(q_segment_ids, kv_segment_ids):
                mask = q_segment_ids[:, :, None] == kv_segment_ids[:, None, :]
                return jnp.where(mask, 0, -jnp.inf)[:, None, :, :]

        def program(qs, ks, vs, dos, qkw, kkw):
            out = ref.ring_attention(qs, ks, vs, axis_name="sp", bias_fn=bias_fn, bias_q_kwargs=qkw,
                                     bias_kv_kwargs=kkw, block_impl=block_impl)
            return (out,) + tuple(tail(dos))

        qkw = {} if q_seg is None else {"q_segment_ids": q_seg}
        kkw = {} if kv_seg is None else {"kv_segment_ids": kv_seg}
        run = standin.shard_map(program, mesh, in_specs=(spec,) * 6, out_specs=spec)
        out, L, dq, dk, dv = run(q, k, v, do, qkw, kkw)
    else:
        assert q_seg is kv_seg or np.array_equal(q_seg, kv_seg), "self attention: one set of segment ids"
        out = ref.ring_self_attention(q, k, v, mesh, spec, causal=causal, segment_ids=q_seg, positions=q_pos,
                                      prefix_mask=q_pre, block_impl=block_impl)
        ctx = standin.LAST_CTX
        parts = standin.run_spmd(ctx, tail, [[np.array_split(do, nranks, axis=1)[r]] for r in range(nranks)])
        L, dq, dk, dv = (np.concatenate([p[i] for p in parts], axis=1) for i in range(4))
    return {"out": np.asarray(out), "lse": np.transpose(np.asarray(L), (0, 2, 1)), "dq": np.asarray(dq),
            "dk": np.asarray(dk), "dv": np.asarray(dv)}
