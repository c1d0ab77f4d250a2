"""ra_fwd_block_static: the forward block for hosts that cannot allocate device memory.

Some callers of this library run where a driver allocation is off the table: an XLA / JAX
FFI custom-call handler works while XLA's allocator already holds almost all of the GPU's
memory, and a serving process may have given every free byte to its own arena.  For them
the library offers the tensor-core forward block with its scratch (per-tile mask
summaries) in a fixed array inside the library image.  This file checks, through the
C ABI, that it returns what ra_fwd_block returns, on two calls in a row (the second call
reuses the array the first one wrote and continues from the first one's state), and that
a problem larger than the fixed array is refused before anything runs.

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


@pytest.mark.gpu
def test_static_scratch_forward_matches_allocating_forward_twice():
    L = _lib()
    lib = L.lib
    b, h, lq, lk, d = 2, 2, 512, 768, 128
    g = torch.Generator().manual_seed(7)
    mk = lambda n: torch.randn((b, n, h, d), generator=g).to(torch.bfloat16).cuda()
    q = mk(lq)
    blocks = [(mk(lk), mk(lk)) for _ in range(2)]  # two K/V blocks, as two ring steps would bring
    qpos = (torch.arange(lq, dtype=torch.int32) + 2 * lk - lq).expand(b, lq).contiguous().cuda()
    seg_q = torch.randint(0, 2, (b, lq), generator=g, dtype=torch.int32).cuda()
    sh = L.RaShape(b, h, lq, lk, d, d, L.RA_DTYPE_BF16, 1 / math.sqrt(d))
    assert lib.ra_set_impl(L.RA_IMPL_TCGEN05) == 0
    results = {}
    for name, fn in (("alloc", lib.ra_fwd_block), ("static", lib.ra_fwd_block_static)):
        o = torch.empty((b, h, lq, d), device="cuda")
        m = torch.empty((b, h, lq), device="cuda")
        l = torch.empty((b, h, lq), device="cuda")
        for step, (k, v) in enumerate(blocks):  # two calls in a row
            kpos = (torch.arange(lk, dtype=torch.int32) + step * lk).expand(b, lk).contiguous().cuda()
            seg_k = torch.randint(0, 2, (b, lk), generator=torch.Generator().manual_seed(step), dtype=torch.int32).cuda()
            mod = L.RaScoreMod()
            mod.kinds = L.RA_MOD_CAUSAL | L.RA_MOD_SEGMENT
            mod.q_pos, mod.kv_pos = qpos.data_ptr(), kpos.data_ptr()
            mod.q_seg, mod.kv_seg = seg_q.data_ptr(), seg_k.data_ptr()
            rc = _call(fn, sh, q, k, v, mod, o, m, l, int(step == 0))
            assert rc == 0, lib.ra_last_error_string().decode()
            torch.cuda.synchronize()
        results[name] = (o.cpu().double().numpy(), m.cpu().double().numpy(), l.cpu().double().numpy())
    assert lib.ra_set_impl(L.RA_IMPL_AUTO) == 0
    bits = C.c_uint32(0)
    assert lib.ra_device_status(C.byref(bits)) == 0, hex(bits.value)
    for got, want, name in zip(results["static"], results["alloc"], "oml"):
        np.testing.assert_array_equal(np.isneginf(got), np.isneginf(want), err_msg=name)
        ok = np.isfinite(want)
        assert ok.any()
        err = np.abs(got[ok] - want[ok])
        assert np.all(err <= BF16_ATOL + BF16_RTOL * np.abs(want[ok])), (name, err.max())


def test_static_scratch_refuses_more_tiles_than_it_holds():
    """Checked on the host before any launch, so it needs no GPU: pointers are never read."""
    L = _lib()
    lib = L.lib
    b, lq, lk, d = 3, 128 * 4096, 128 * 4096, 128  # 3 * 8192 tiles > RA_STATIC_MAX_TILES
    t = L.RaTensor(0x10000, lq * d, d, d)
    one = C.c_void_p(0x10000)
    sh = L.RaShape(b, 1, lq, lk, d, d, L.RA_DTYPE_BF16, 1.0)
    rc = lib.ra_fwd_block_static(C.byref(sh), C.byref(t), C.byref(t), C.byref(t), None, one, one, one, 1, None)
    assert rc == -41, (rc, lib.ra_last_error_string().decode())
    assert "exceeds" in lib.ra_last_error_string().decode()
    sh32 = L.RaShape(1, 1, 128, 128, d, d, L.RA_DTYPE_F32, 1.0)
    rc = lib.ra_fwd_block_static(C.byref(sh32), C.byref(t), C.byref(t), C.byref(t), None, one, one, one, 1, None)
    assert rc == -40
