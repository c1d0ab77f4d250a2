"""ra_fwd_block_static: the forward block for hosts that cannot allocate device memory.

Some callers of this library run where a driver allocation is off the table: an XLA / JAX
FFI custom-call handler works while XLA's allocator already holds almost all of the GPU's
memory, and a serving process may have given every free byte to its own arena.  For them
the library offers the tensor-core forward block with its scratch (per-tile mask
summaries) in a fixed array inside the library image.  This file checks, through the
C ABI, that it returns bit for bit what ra_fwd_block returns, on two calls in a row (the
second call reuses the array the first one wrote and continues from the first one's state)
and then on a problem of another shape, that both agree with the CPU oracle, and that a
masked problem larger than the fixed array is refused before anything runs.

The file name makes pytest collect it after every other test.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from tests.util import BF16_ATOL, BF16_RTOL


def _lib():
    from ring_attention_b200 import _lib

    return _lib


def _call(fn, sh, q, k, v, mod, o, m, l, first):
    L = _lib()
    tv = lambda t: C.byref(L.RaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)))
    return fn(C.byref(sh), tv(q), tv(k), tv(v), C.byref(mod), o.data_ptr(), m.data_ptr(), l.data_ptr(), first, None)


def _run_blocks(fn, b, h, lq, lk, d, n_blocks, seed):
    """`n_blocks` calls in a row on one carried state, as ring steps would make them; returns
    the inputs (for the oracle) and the final (o, m, l)."""
    L = _lib()
    g = torch.Generator().manual_seed(seed)
    mk = lambda n: torch.randn((b, n, h, d), generator=g).to(torch.bfloat16).cuda()
    q = mk(lq)
    blocks = [(mk(lk), mk(lk)) for _ in range(n_blocks)]
    qpos = (torch.arange(lq, dtype=torch.int32) + n_blocks * lk - lq).expand(b, lq).contiguous().cuda()
    seg_q = torch.randint(0, 2, (b, lq), generator=g, dtype=torch.int32).cuda()
    sh = L.RaShape(b, h, lq, lk, d, d, L.RA_DTYPE_BF16, 1 / math.sqrt(d))
    o = torch.empty((b, h, lq, d), device="cuda")
    m = torch.empty((b, h, lq), device="cuda")
    l = torch.empty((b, h, lq), device="cuda")
    kv_meta = []
    for step, (k, v) in enumerate(blocks):
        kpos = (torch.arange(lk, dtype=torch.int32) + step * lk).expand(b, lk).contiguous().cuda()
        seg_k = torch.randint(0, 2, (b, lk), generator=torch.Generator().manual_seed(100 * seed + step), dtype=torch.int32).cuda()
        mod = L.RaScoreMod()
        mod.kinds = L.RA_MOD_CAUSAL | L.RA_MOD_SEGMENT
        mod.q_pos, mod.kv_pos = qpos.data_ptr(), kpos.data_ptr()
        mod.q_seg, mod.kv_seg = seg_q.data_ptr(), seg_k.data_ptr()
        rc = _call(fn, sh, q, k, v, mod, o, m, l, int(step == 0))
        assert rc == 0, L.lib.ra_last_error_string().decode()
        torch.cuda.synchronize()
        kv_meta.append((kpos, seg_k))
    return (q, blocks, qpos, seg_q, kv_meta), (o, m, l)


@pytest.mark.gpu
def test_static_scratch_forward_matches_allocating_forward_twice():
    from oracle import oracle as O

    L = _lib()
    lib = L.lib
    assert lib.ra_set_impl(L.RA_IMPL_TCGEN05) == 0
    # Two calls in a row on one state, then a third problem with another batch size and block
    # length: the split of the fixed array between query-side and key-side summaries moves, so
    # a stale or misplaced entry would be read and would change which tiles are skipped.
    for b, h, lq, lk, d, n_blocks, seed in ((2, 2, 512, 768, 128, 2, 7), (3, 1, 384, 1280, 128, 1, 8)):
        _, want = _run_blocks(lib.ra_fwd_block, b, h, lq, lk, d, n_blocks, seed)
        inputs, got = _run_blocks(lib.ra_fwd_block_static, b, h, lq, lk, d, n_blocks, seed)
        # same kernel, same inputs, same summaries: the results must be the same bits
        for x, y, name in zip(got, want, "oml"):
            assert torch.equal(x, y) or torch.equal(torch.nan_to_num(x, nan=7.0), torch.nan_to_num(y, nan=7.0)), name
        # and both are right: the oracle's block updates (ring.py:58-76) on the same inputs
        q, blocks, qpos, seg_q, kv_meta = inputs
        f = lambda t: t.to(torch.float64).cpu().numpy()
        o_ref = np.zeros((b, h, lq, d))
        m_ref = np.full((b, h, lq), -np.inf)
        l_ref = np.zeros((b, h, lq))
        for (k, v), (kpos, seg_k) in zip(blocks, kv_meta):
            bias = O.score_mod_bias(b, h, q_positions=f(qpos).astype(np.int64), kv_positions=f(kpos).astype(np.int64),
                                    q_segment_ids=f(seg_q).astype(np.int64), kv_segment_ids=f(seg_k).astype(np.int64),
                                    causal=True)
            o_ref, m_ref, l_ref = O.fwd_block(f(q).transpose(0, 2, 1, 3), f(k).transpose(0, 2, 1, 3),
                                              f(v).transpose(0, 2, 1, 3), bias, o_ref, m_ref, l_ref, 1 / math.sqrt(d))
        with np.errstate(invalid="ignore", divide="ignore"):
            out_ref, L_ref = O.finalize(o_ref, m_ref, l_ref)
            o_got, m_got, l_got = (f(t) for t in got)
            out_got = o_got / l_got[..., None]
            L_got = m_got + np.log(l_got)
        np.testing.assert_array_equal(np.isnan(out_got), np.isnan(out_ref))
        ok = np.isfinite(out_ref)
        assert ok.any()
        err = np.abs(out_got[ok] - out_ref[ok])
        assert np.all(err <= BF16_ATOL + BF16_RTOL * np.abs(out_ref[ok])), err.max()
        okL = np.isfinite(L_ref)
        np.testing.assert_array_equal(np.isfinite(L_got), okL)
        assert np.all(np.abs(L_got[okL] - L_ref[okL]) <= BF16_ATOL + BF16_RTOL * np.abs(L_ref[okL]))
    assert lib.ra_set_impl(L.RA_IMPL_AUTO) == 0
    bits = C.c_uint32(0)
    assert lib.ra_device_status(C.byref(bits)) == 0, hex(bits.value)


def test_static_scratch_refuses_more_tiles_than_it_holds():
    """Checked on the host before any launch, so it needs no GPU: pointers are never read."""
    L = _lib()
    lib = L.lib
    b, lq, lk, d = 3, 128 * 4096, 128 * 4096, 128  # 3 * 8192 tiles > RA_STATIC_MAX_TILES
    t = L.RaTensor(0x10000, lq * d, d, d)
    one = C.c_void_p(0x10000)
    sh = L.RaShape(b, 1, lq, lk, d, d, L.RA_DTYPE_BF16, 1.0)
    mod = L.RaScoreMod()  # a mask that reads the tile summaries (the pointers are never read: refused first)
    mod.kinds = L.RA_MOD_CAUSAL
    mod.q_pos = mod.kv_pos = 0x10000
    rc = lib.ra_fwd_block_static(C.byref(sh), C.byref(t), C.byref(t), C.byref(t), C.byref(mod), one, one, one, 1, None)
    assert rc == -41, (rc, lib.ra_last_error_string().decode())
    assert "exceeds" in lib.ra_last_error_string().decode()
    sh32 = L.RaShape(1, 1, 128, 128, d, d, L.RA_DTYPE_F32, 1.0)
    rc = lib.ra_fwd_block_static(C.byref(sh32), C.byref(t), C.byref(t), C.byref(t), None, one, one, one, 1, None)
    assert rc == -40
