"""Ring-handle behaviour that needs a GPU but no peer: the bounded wait's time-out path and
reserving the handle's buffers ahead of time.  The time-out is produced the allowed way: a
wait on a counter that nothing advances, with a 1 ms bound; the kernel returns and the host
reads the status.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_that_nothing_satisfies_times_out_reports_and_aborts_the_ring():
    import ring_attention_b200 as ra
    from ring_attention_b200 import _lib

    assert ra.device_status() == 0
    ring = ra.Ring(0, 1)
    assert not ring.aborted
    ring.set_wait_ms(1)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(_lib.lib.ra_ring_probe_wait(ring.handle, stream))
    bits = C.c_uint32(0)
    rc = _lib.lib.ra_device_status(C.byref(bits))
    assert rc == _lib.RA_ERR_DEVICE_STATUS, rc
    assert bits.value & (1 << 16), hex(bits.value)
    assert b"bounded wait" in _lib.lib.ra_last_error_string()
    # reading clears the word; the ring stays aborted (its later waits return at once and its
    # flag stores are suppressed) until it is destroyed
    assert ra.device_status() == 0
    assert ring.aborted
    _lib.check(_lib.lib.ra_ring_probe_wait(ring.handle, stream))  # returns immediately: already aborted
    assert ra.device_status() == 0
    ring.destroy()
    # the context is intact: a fresh ring computes
    q = torch.randn((1, 256, 2, 128), device="cuda").to(torch.bfloat16)
    out = ra.ring_attention(q, q, q, ra.Ring(0, 1))
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert _lib.lib.ra_ring_set_wait_ms(None, 5) == -30 and _lib.lib.ra_ring_probe_wait(None, None) == -30


def test_reserved_ring_calls_allocate_nothing():
    import ring_attention_b200 as ra
    from ring_attention_b200 import _lib
    from ring_attention_b200._lib import RaScoreMod, RaShape, RaTensor, check, lib

    b, s, h, d = 2, 1024, 2, 128
    ring = ra.Ring(0, 1)
    q, k, v, do = (torch.randn((b, s, h, d), device="cuda").to(torch.bfloat16) for _ in range(4))
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    lse = torch.empty((b, h, s), dtype=torch.float32, device="cuda")
    pos = torch.arange(s, dtype=torch.int32, device="cuda").expand(b, s).contiguous()
    mod = RaScoreMod()
    mod.kinds = _lib.RA_MOD_CAUSAL
    mod.q_pos = mod.kv_pos = pos.data_ptr()
    sh = RaShape(b, h, s, s, d, d, _lib.RA_DTYPE_BF16, 1 / math.sqrt(d))
    tv = lambda t: C.byref(RaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # a smaller problem first, so that the kernels are loaded; then reserve the full shape
    small = RaShape(b, h, 256, 256, d, d, _lib.RA_DTYPE_BF16, 1 / math.sqrt(d))
    check(lib.ra_ring_fwd(ring.handle, C.byref(small), tv(q), tv(k), tv(v), C.byref(mod), tv(out), lse.data_ptr(), stream))
    check(lib.ra_ring_bwd(ring.handle, C.byref(small), tv(q), tv(k), tv(v), tv(out), lse.data_ptr(), tv(do), C.byref(mod),
                          tv(dq), tv(dk), tv(dv), stream))
    check(lib.ra_ring_reserve(ring.handle, C.byref(sh), C.byref(mod), 1))
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(2):
        check(lib.ra_ring_fwd(ring.handle, C.byref(sh), tv(q), tv(k), tv(v), C.byref(mod), tv(out), lse.data_ptr(), stream))
        check(lib.ra_ring_bwd(ring.handle, C.byref(sh), tv(q), tv(k), tv(v), tv(out), lse.data_ptr(), tv(do), C.byref(mod),
                              tv(dq), tv(dk), tv(dv), stream))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"device memory in use grew by {free0 - free1} bytes inside reserved ring calls"
    assert ra.device_status() == 0
    # the timing diagnostics of the last call: one block launch per direction on a ring of one,
    # no waits for transfers, nothing pushed
    ring.set_timing(True)
    check(lib.ra_ring_fwd(ring.handle, C.byref(sh), tv(q), tv(k), tv(v), C.byref(mod), tv(out), lse.data_ptr(), stream))
    check(lib.ra_ring_bwd(ring.handle, C.byref(sh), tv(q), tv(k), tv(v), tv(out), lse.data_ptr(), tv(do), C.byref(mod),
                          tv(dq), tv(dk), tv(dv), stream))
    for back in (False, True):
        blocks, waits = ring.last_timeline(back)
        assert len(blocks) == 1 and waits == [] and blocks[0][1] > blocks[0][0] >= 0, (blocks, waits)
        total, exposed = ring.last_timing(back)
        assert total >= blocks[0][1] - blocks[0][0] > 0 and exposed == 0
        assert abs(ring.last_block_ms(back)[0] - (blocks[0][1] - blocks[0][0])) < 1e-3
        assert ring.last_push(back) == (0.0, 0.0)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2).float(), k.transpose(1, 2).float(), v.transpose(1, 2).float(), is_causal=True).transpose(1, 2)
    assert (out.float() - ref).abs().max() < 3e-2
    ring.destroy()
