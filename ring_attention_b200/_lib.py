"""ctypes binding of libring_attention_b200.so (declared in include/ring_attention_b200.h).

There is no fallback: if the shared library is missing the import fails, and every
compute call needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# RA_LIB_PATH: load a library built elsewhere (another build of the same sources) instead of the in-tree one
LIB_PATH = os.environ.get("RA_LIB_PATH") or os.path.join(_HERE, "libring_attention_b200.so")

RA_DTYPE_F32, RA_DTYPE_BF16 = 0, 1
RA_MOD_CAUSAL, RA_MOD_SEGMENT, RA_MOD_PREFIX, RA_MOD_ALIBI, RA_MOD_WINDOW, RA_MOD_DENSE = 1, 2, 4, 8, 16, 32
RA_MOD_STRICT_NAN = 64
RA_IMPL_AUTO, RA_IMPL_SIMT, RA_IMPL_TCGEN05 = 0, 1, 2
RA_UNIQUE_ID_BYTES = 128


class RaTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_l", C.c_int64), ("stride_h", C.c_int64)]


class RaShape(C.Structure):
    _fields_ = [
        ("b", C.c_int32), ("h", C.c_int32), ("lq", C.c_int32), ("lk", C.c_int32),
        ("dk", C.c_int32), ("dv", C.c_int32), ("dtype", C.c_int32), ("sm_scale", C.c_float),
    ]


class RaScoreMod(C.Structure):
    _fields_ = [
        ("kinds", C.c_uint32), ("window", C.c_int32),
        ("q_pos", C.c_void_p), ("kv_pos", C.c_void_p), ("q_seg", C.c_void_p), ("kv_seg", C.c_void_p),
        ("q_prefix", C.c_void_p), ("kv_prefix", C.c_void_p), ("alibi_slopes", C.c_void_p),
        ("bias", C.c_void_p), ("bias_stride_b", C.c_int64), ("bias_stride_h", C.c_int64),
        ("bias_stride_q", C.c_int64),
    ]


_P = C.POINTER
_SIGNATURES = {
    "ra_version": (C.c_int, []),
    "ra_last_error_string": (C.c_char_p, []),
    "ra_set_impl": (C.c_int, [C.c_int]),
    "ra_last_impl": (C.c_int, []),
    "ra_launch_count": (C.c_int64, []),
    "ra_device_status": (C.c_int, [_P(C.c_uint32)]),
    "ra_fwd_block": (C.c_int, [_P(RaShape), _P(RaTensor), _P(RaTensor), _P(RaTensor), _P(RaScoreMod),
                               C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "ra_fwd_block_static": (C.c_int, [_P(RaShape), _P(RaTensor), _P(RaTensor), _P(RaTensor), _P(RaScoreMod),
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "ra_fwd_finalize": (C.c_int, [_P(RaShape), C.c_void_p, C.c_void_p, C.c_void_p, _P(RaTensor),
                                  C.c_void_p, C.c_void_p]),
    "ra_bwd_delta": (C.c_int, [_P(RaShape), _P(RaTensor), _P(RaTensor), C.c_void_p, C.c_void_p]),
    "ra_bwd_block": (C.c_int, [_P(RaShape), _P(RaTensor), _P(RaTensor), _P(RaTensor), _P(RaScoreMod),
                               C.c_void_p, C.c_void_p, _P(RaTensor), C.c_void_p, C.c_void_p, C.c_void_p,
                               C.c_void_p]),
    "ra_cast_from_f32": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, _P(RaTensor),
                                   C.c_int32, C.c_void_p]),
    "ra_ring_unique_id": (C.c_int, [C.c_void_p]),
    "ra_ring_create": (C.c_int, [C.c_int32, C.c_int32, C.c_void_p, _P(C.c_void_p)]),
    "ra_ring_destroy": (C.c_int, [C.c_void_p]),
    "ra_ring_rank": (C.c_int, [C.c_void_p]),
    "ra_ring_size": (C.c_int, [C.c_void_p]),
    "ra_ring_source": (C.c_int, [C.c_int32, C.c_int32, C.c_int32]),
    "ra_ring_fwd": (C.c_int, [C.c_void_p, _P(RaShape), _P(RaTensor), _P(RaTensor), _P(RaTensor),
                              _P(RaScoreMod), _P(RaTensor), C.c_void_p, C.c_void_p]),
    "ra_ring_bwd": (C.c_int, [C.c_void_p, _P(RaShape), _P(RaTensor), _P(RaTensor), _P(RaTensor),
                              _P(RaTensor), C.c_void_p, _P(RaTensor), _P(RaScoreMod), _P(RaTensor),
                              _P(RaTensor), _P(RaTensor), C.c_void_p]),
    "ra_ring_plan_create": (C.c_int, [C.c_void_p, _P(RaShape), _P(RaScoreMod), C.c_void_p, _P(C.c_void_p)]),
    "ra_ring_plan_destroy": (None, [C.c_void_p]),
    "ra_ring_plan_need": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32]),
    "ra_ring_plan_rows": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, _P(C.c_int32)]),
    "ra_ring_use_plan": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ra_ring_rotate": (C.c_int, [C.c_void_p, C.c_int32, _P(C.c_void_p), _P(C.c_void_p), _P(C.c_int64),
                                 C.c_void_p]),
    "ra_ring_transport": (C.c_int, [C.c_void_p]),
    "ra_ring_reserve": (C.c_int, [C.c_void_p, _P(RaShape), _P(RaScoreMod), C.c_int32]),
    "ra_ring_set_wait_ms": (C.c_int, [C.c_void_p, C.c_int32]),
    "ra_ring_aborted": (C.c_int, [C.c_void_p]),
    "ra_ring_probe_wait": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ra_ring_set_timing": (C.c_int, [C.c_void_p, C.c_int32]),
    "ra_ring_last_timing": (C.c_int, [C.c_void_p, C.c_int32, _P(C.c_float), _P(C.c_float)]),
    "ra_ring_last_block_ms": (C.c_int, [C.c_void_p, C.c_int32, _P(C.c_float), _P(C.c_int32)]),
    "ra_ring_last_push": (C.c_int, [C.c_void_p, C.c_int32, _P(C.c_double), _P(C.c_float)]),
    "ra_ring_last_timeline": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, _P(C.c_float), _P(C.c_int32), _P(C.c_float),
                                        _P(C.c_int32)]),
}

EXPORTS = tuple(_SIGNATURES)


class RingAttentionError(RuntimeError):
    pass


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python ring_attention_b200/build.py` "
            "(needs nvcc; there is no CPU or PyTorch fallback)"
        )
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


RA_ERR_DEVICE_STATUS = 3


def device_status() -> int:
    """Synchronises the current device and returns (and clears) its kernel status word: 0 when no
    bounded wait inside a kernel has run out since the last read (bits 0-10: the tcgen05 kernels'
    own waits; bit 16: a ring's wait for a peer)."""
    bits = C.c_uint32(0)
    rc = lib.ra_device_status(C.byref(bits))
    if rc not in (0, RA_ERR_DEVICE_STATUS):
        check(rc)
    return int(bits.value)


def check(rc: int) -> None:
    """Raise with the library's own message when a call failed."""
    if rc != 0:
        msg = lib.ra_last_error_string()
        raise RingAttentionError(f"ring_attention_b200 error {rc}: {msg.decode() if msg else ''}")
