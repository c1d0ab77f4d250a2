"""Host side of the engine: the reference's Python surface over the C ABI.

Mirrors ring_attention/ring.py of jondeaton/ring-attention-jax-pallas:
`ring_attention` (ring.py:246-325), `ring_self_attention` (ring.py:328-449), the
custom-VJP pair (ring.py:214-243) and the block plug point `fwd_block` / `bwd_block`
(ring_kernel.py:123-140, 202-219).  Arrays are torch CUDA tensors; one process drives one
GPU and holds one shard, so what `shard_map` did is the caller's process layout and
`axis_name` resolves to a `Ring` (see mesh.py).

All arithmetic runs in libring_attention_b200.so.  PyTorch provides device memory,
streams and autograd bookkeeping only.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Callable, Optional

import torch

from . import _lib
from ._lib import RaScoreMod, RaShape, RaTensor, check, lib
from .mesh import Mesh, PartitionSpec, Ring, resolve_axis

_IMPLS = {
    "cuda": _lib.RA_IMPL_AUTO,
    "simt": _lib.RA_IMPL_SIMT,
    "tcgen05": _lib.RA_IMPL_TCGEN05,
    # the reference's two values keep working and mean "let the engine choose"
    "pallas": _lib.RA_IMPL_AUTO,
    "jax": _lib.RA_IMPL_AUTO,
}


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.RA_DTYPE_F32
    if t.dtype == torch.bfloat16:
        return _lib.RA_DTYPE_BF16
    raise TypeError(f"ring_attention_b200 takes float32 or bfloat16 tensors, got {t.dtype}")


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.RingAttentionError("ring_attention_b200 needs CUDA tensors (there is no CPU path)")


def _blhd(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def _view_blhd(t: torch.Tensor) -> RaTensor:
    """[b, l, h, d] tensor -> ra_tensor_t."""
    return RaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _view_bhld(t: torch.Tensor) -> RaTensor:
    """[b, h, l, d] tensor -> ra_tensor_t."""
    return RaTensor(t.data_ptr(), t.stride(0), t.stride(2), t.stride(1))


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


# ----------------------------------------------------------------------------------------
# Score-mods: the bias_fn variants that are compiled into the kernels.
# ----------------------------------------------------------------------------------------
class ScoreMod:
    """A `bias_fn` the kernels evaluate themselves instead of reading a dense tile.

    It is also an ordinary callable with the reference's protocol
    `bias_fn(**bias_q_kwargs, **bias_kv_kwargs) -> [b, h or 1, lq, lk]` (ring.py:107), so the
    same object can be handed to the dense-tile path.  Keyword names are those of the
    reference's built-in mask (ring.py:376-383): q_/kv_ + segment_ids, positions,
    prefix_mask.  Segment and prefix masking switch on when those arrays are passed.
    """

    def __init__(self, causal: bool = False, alibi_slopes: Optional[torch.Tensor] = None, window: int = 0,
                 strict_nan: bool = False):
        self.causal = bool(causal)
        self.alibi_slopes = alibi_slopes
        self.window = int(window)
        # True: a query row that sees no key poisons dQ of that row and dK, dV of its whole
        # (batch, head) with NaN, as the reference's arithmetic does (ring.py:146); False
        # (default): such rows contribute nothing to the gradients
        self.strict_nan = bool(strict_nan)

    def kinds(self, q_kwargs: dict, kv_kwargs: dict) -> int:
        k = 0
        if q_kwargs.get("q_segment_ids") is not None:
            k |= _lib.RA_MOD_SEGMENT
        if self.causal:
            k |= _lib.RA_MOD_CAUSAL
        elif q_kwargs.get("q_prefix_mask") is not None:
            k |= _lib.RA_MOD_PREFIX
        if self.alibi_slopes is not None:
            k |= _lib.RA_MOD_ALIBI
        if self.window:
            k |= _lib.RA_MOD_WINDOW
        if self.strict_nan:
            k |= _lib.RA_MOD_STRICT_NAN
        return k

    def __call__(self, q_segment_ids=None, kv_segment_ids=None, q_positions=None, kv_positions=None,
                 q_prefix_mask=None, kv_prefix_mask=None):
        mask = None

        def conj(a, b):
            return b if a is None else a & b

        rel = None
        if q_positions is not None:
            rel = q_positions[:, :, None].long() - kv_positions[:, None, :].long()
        if q_segment_ids is not None:
            mask = conj(mask, q_segment_ids[:, :, None] == kv_segment_ids[:, None, :])
        if self.causal:
            mask = conj(mask, rel >= 0)
        elif q_prefix_mask is not None:
            pre = q_prefix_mask[:, :, None].bool() & kv_prefix_mask[:, None, :].bool()
            mask = conj(mask, pre | (rel >= 0))
        if self.window:
            mask = conj(mask, rel < self.window)
        ref = q_positions if q_positions is not None else q_segment_ids
        kref = kv_positions if kv_positions is not None else kv_segment_ids
        b, lq, lk = ref.shape[0], ref.shape[1], kref.shape[1]
        if self.alibi_slopes is not None:
            bias = -self.alibi_slopes.float()[None, :, None, None] * rel[:, None].float()
        else:
            bias = torch.zeros((b, 1, lq, lk), dtype=torch.float32, device=ref.device)
        if mask is not None:
            bias = torch.where(mask[:, None], bias, torch.full_like(bias, float("-inf")))
        return bias


def _i32(t):
    if t is None:
        return None
    return t.to(torch.int32).contiguous()


def _u8(t):
    if t is None:
        return None
    return t.to(torch.uint8).contiguous()


class _ModArgs:
    """Owns the converted per-token arrays and the ra_score_mod_t that points at them."""

    def __init__(self, bias_fn, q_kwargs, kv_kwargs, heads: int):
        self.struct = None
        self.keep = []
        if bias_fn is None:
            return
        assert isinstance(bias_fn, ScoreMod)
        m = RaScoreMod()
        m.kinds = bias_fn.kinds(q_kwargs, kv_kwargs)
        m.window = bias_fn.window

        def put(field, t):
            if t is not None:
                _need_cuda(t)
                self.keep.append(t)
                setattr(m, field, t.data_ptr())

        put("q_pos", _i32(q_kwargs.get("q_positions")))
        put("kv_pos", _i32(kv_kwargs.get("kv_positions")))
        put("q_seg", _i32(q_kwargs.get("q_segment_ids")))
        put("kv_seg", _i32(kv_kwargs.get("kv_segment_ids")))
        put("q_prefix", _u8(q_kwargs.get("q_prefix_mask")))
        put("kv_prefix", _u8(kv_kwargs.get("kv_prefix_mask")))
        if bias_fn.alibi_slopes is not None:
            s = bias_fn.alibi_slopes.to(torch.float32).contiguous()
            if s.numel() != heads:
                raise ValueError(f"alibi_slopes has {s.numel()} entries for {heads} heads")
            put("alibi_slopes", s)
        self.struct = m

    def ref(self):
        return C.byref(self.struct) if self.struct is not None else None


def _dense_mod(bias: Optional[torch.Tensor], b: int, h: int, lq: int, lk: int):
    """ra_score_mod_t for a materialised bias [b, h or 1, lq, lk] (ring.py:60-61, 409)."""
    if bias is None:
        return None, None
    bias = bias.to(torch.float32)
    if bias.dim() == 3:
        bias = bias[:, None]
    if bias.shape[0] != b or bias.shape[1] not in (1, h) or bias.shape[2] != lq or bias.shape[3] != lk:
        raise ValueError(f"bias shape {tuple(bias.shape)} does not match [b={b}, h={h} or 1, {lq}, {lk}]")
    bias = bias.contiguous()
    m = RaScoreMod()
    m.kinds = _lib.RA_MOD_DENSE
    m.bias = bias.data_ptr()
    m.bias_stride_b = bias.stride(0)
    m.bias_stride_h = 0 if bias.shape[1] == 1 else bias.stride(1)
    m.bias_stride_q = bias.stride(2)
    return m, bias


def _shape(b, h, lq, lk, dk, dv, dtype, sm_scale) -> RaShape:
    return RaShape(b, h, lq, lk, dk, dv, dtype, float(sm_scale))


def _set_impl(block_impl: str):
    if block_impl not in _IMPLS:
        raise ValueError(block_impl)  # ring.py:311-312
    check(lib.ra_set_impl(_IMPLS[block_impl]))


# ----------------------------------------------------------------------------------------
# Block plug point: ring_kernel.py:123-140 (fwd_block) and :202-219 (bwd_block); [b,h,l,d].
# ----------------------------------------------------------------------------------------
def fwd_block(q, k, v, bias, o, m, l, sm_scale: float, block_impl: str = "cuda"):
    """One online-softmax update; returns new (o, m, l) like ring.py:58-76.

    o is carried in float32 whatever the input dtype (the reference carries it in
    q.dtype, ring.py:124; float32 is a superset and keeps bf16 runs accurate).
    """
    _need_cuda(q, k, v, o, m, l)
    _set_impl(block_impl)
    b, h, lq, dk = q.shape
    lk, dv = v.shape[2], v.shape[3]
    q, k, v = _blhd(q), _blhd(k), _blhd(v)
    o2 = o.to(torch.float32).clone().contiguous()
    m2 = m.to(torch.float32).clone().contiguous()
    l2 = l.to(torch.float32).clone().contiguous()
    mod, keep = _dense_mod(bias, b, h, lq, lk)
    sh = _shape(b, h, lq, lk, dk, dv, _dtype_code(q), sm_scale)
    check(lib.ra_fwd_block(C.byref(sh), C.byref(_view_bhld(q)), C.byref(_view_bhld(k)), C.byref(_view_bhld(v)),
                           C.byref(mod) if mod is not None else None, _ptr(o2), _ptr(m2), _ptr(l2), 0, _stream()))
    del keep
    return o2, m2, l2


def bwd_block(q, k, v, bias, o, L, do, sm_scale: float, block_impl: str = "cuda"):
    """Block VJP; returns float32 (dq, dk, dv) like ring.py:140-157."""
    _need_cuda(q, k, v, o, L, do)
    _set_impl(block_impl)
    b, h, lq, dk = q.shape
    lk, dv = v.shape[2], v.shape[3]
    q, k, v, o, do = _blhd(q), _blhd(k), _blhd(v), _blhd(o), _blhd(do)
    L = L.to(torch.float32).contiguous()
    delta = torch.empty((b, h, lq), dtype=torch.float32, device=q.device)
    dq = torch.zeros((b, h, lq, dk), dtype=torch.float32, device=q.device)
    dkk = torch.zeros((b, h, lk, dk), dtype=torch.float32, device=q.device)
    dvv = torch.zeros((b, h, lk, dv), dtype=torch.float32, device=q.device)
    mod, keep = _dense_mod(bias, b, h, lq, lk)
    sh = _shape(b, h, lq, lk, dk, dv, _dtype_code(q), sm_scale)
    check(lib.ra_bwd_delta(C.byref(sh), C.byref(_view_bhld(o)), C.byref(_view_bhld(do)), _ptr(delta), _stream()))
    check(lib.ra_bwd_block(C.byref(sh), C.byref(_view_bhld(q)), C.byref(_view_bhld(k)), C.byref(_view_bhld(v)),
                           C.byref(mod) if mod is not None else None, _ptr(L), _ptr(delta),
                           C.byref(_view_bhld(do)), _ptr(dq), _ptr(dkk), _ptr(dvv), _stream()))
    del keep
    return dq, dkk, dvv


# ----------------------------------------------------------------------------------------
# Ring forward / backward.  Fused (ra_ring_fwd / ra_ring_bwd) when bias_fn is None or a
# ScoreMod; otherwise the reference's own schedule on the host with a dense tile per step.
# ----------------------------------------------------------------------------------------
def _rotate(ring: Ring, tensors):
    """ppermute i -> i+1 of a list of dense tensors (ring.py:41-55); returns new tensors."""
    srcs = [t.contiguous() for t in tensors]
    dsts = [torch.empty_like(t) for t in srcs]
    n = len(srcs)
    if n:
        a = (C.c_void_p * n)(*[t.data_ptr() for t in srcs])
        d = (C.c_void_p * n)(*[t.data_ptr() for t in dsts])
        nb = (C.c_int64 * n)(*[t.numel() * t.element_size() for t in srcs])
        check(lib.ra_ring_rotate(ring.handle, n, a, d, nb, _stream()))
    return dsts


def _rotate_kwargs(ring: Ring, kw: dict):
    keys = [k for k, v in kw.items() if v is not None]
    out = dict(kw)
    for k, t in zip(keys, _rotate(ring, [kw[k] for k in keys])):
        out[k] = t
    return out


def _fused_fwd(ring, q, k, v, sm_scale, bias_fn, q_kwargs, kv_kwargs):
    b, lq, h, dk = q.shape
    lk, dv = k.shape[1], v.shape[3]
    out = torch.empty((b, lq, h, dv), dtype=q.dtype, device=q.device)
    lse = torch.empty((b, h, lq), dtype=torch.float32, device=q.device)
    mod = _ModArgs(bias_fn, q_kwargs, kv_kwargs, h)
    sh = _shape(b, h, lq, lk, dk, dv, _dtype_code(q), sm_scale)
    check(lib.ra_ring_fwd(ring.handle, C.byref(sh), C.byref(_view_blhd(q)), C.byref(_view_blhd(k)),
                          C.byref(_view_blhd(v)), mod.ref(), C.byref(_view_blhd(out)), _ptr(lse), _stream()))
    return out, lse


def _fused_bwd(ring, q, k, v, out, lse, do, sm_scale, bias_fn, q_kwargs, kv_kwargs):
    b, lq, h, dk = q.shape
    lk, dv = k.shape[1], v.shape[3]
    dq, dkk, dvv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    mod = _ModArgs(bias_fn, q_kwargs, kv_kwargs, h)
    sh = _shape(b, h, lq, lk, dk, dv, _dtype_code(q), sm_scale)
    check(lib.ra_ring_bwd(ring.handle, C.byref(sh), C.byref(_view_blhd(q)), C.byref(_view_blhd(k)),
                          C.byref(_view_blhd(v)), C.byref(_view_blhd(out)), _ptr(lse), C.byref(_view_blhd(do)),
                          mod.ref(), C.byref(_view_blhd(dq)), C.byref(_view_blhd(dkk)), C.byref(_view_blhd(dvv)),
                          _stream()))
    return dq, dkk, dvv


def _host_fwd(ring, q, k, v, sm_scale, bias_fn, q_kwargs, kv_kwargs):
    """ring.py:104-137 with the block update done by ra_fwd_block on a dense bias tile."""
    b, lq, h, dk = q.shape
    lk, dv = k.shape[1], v.shape[3]
    dev = q.device
    o = torch.empty((b, h, lq, dv), dtype=torch.float32, device=dev)
    m = torch.empty((b, h, lq), dtype=torch.float32, device=dev)
    l = torch.empty((b, h, lq), dtype=torch.float32, device=dev)
    kc, vc, kvk = k.contiguous(), v.contiguous(), dict(kv_kwargs)
    sh = _shape(b, h, lq, lk, dk, dv, _dtype_code(q), sm_scale)
    for t in range(ring.size):
        bias = bias_fn(**q_kwargs, **kvk)  # ring.py:107
        mod, keep = _dense_mod(bias, b, h, lq, lk)
        check(lib.ra_fwd_block(C.byref(sh), C.byref(_view_blhd(q)), C.byref(_view_blhd(kc)), C.byref(_view_blhd(vc)),
                               C.byref(mod), _ptr(o), _ptr(m), _ptr(l), int(t == 0), _stream()))
        del keep
        if t + 1 < ring.size:  # the reference's last rotation only brings K/V home (ring.py:136)
            kc, vc = _rotate(ring, [kc, vc])  # ring.py:120
            kvk = _rotate_kwargs(ring, kvk)
    out = torch.empty((b, lq, h, dv), dtype=q.dtype, device=dev)
    lse = torch.empty((b, h, lq), dtype=torch.float32, device=dev)
    check(lib.ra_fwd_finalize(C.byref(sh), _ptr(o), _ptr(m), _ptr(l), C.byref(_view_blhd(out)), _ptr(lse), _stream()))
    return out, lse


def _host_bwd(ring, q, k, v, out, lse, do, sm_scale, bias_fn, q_kwargs, kv_kwargs):
    """ring.py:183-211: K, V, dK, dV stay; (q, dq, do, L, delta, q kwargs) travel."""
    b, lq, h, dk = q.shape
    lk, dv = k.shape[1], v.shape[3]
    dev = q.device
    sh = _shape(b, h, lq, lk, dk, dv, _dtype_code(q), sm_scale)
    delta = torch.empty((b, h, lq), dtype=torch.float32, device=dev)
    check(lib.ra_bwd_delta(C.byref(sh), C.byref(_view_blhd(out)), C.byref(_view_blhd(do)), _ptr(delta), _stream()))
    dq = torch.zeros((b, h, lq, dk), dtype=torch.float32, device=dev)  # ring.py:198-200
    dkk = torch.zeros((b, h, lk, dk), dtype=torch.float32, device=dev)
    dvv = torch.zeros((b, h, lk, dv), dtype=torch.float32, device=dev)
    qc, doc, L, qk = q.contiguous(), do.contiguous(), lse.contiguous(), dict(q_kwargs)
    for t in range(ring.size):
        bias = bias_fn(**qk, **kv_kwargs)  # ring.py:185-188
        mod, keep = _dense_mod(bias, b, h, lq, lk)
        check(lib.ra_bwd_block(C.byref(sh), C.byref(_view_blhd(qc)), C.byref(_view_blhd(k)), C.byref(_view_blhd(v)),
                               C.byref(mod), _ptr(L), _ptr(delta), C.byref(_view_blhd(doc)), _ptr(dq), _ptr(dkk),
                               _ptr(dvv), _stream()))
        del keep
        qc, dq, doc, L, delta = _rotate(ring, [qc, dq, doc, L, delta])  # ring.py:195
        qk = _rotate_kwargs(ring, qk)

    def cast(acc, like, n):
        dst = torch.empty_like(like)
        check(lib.ra_cast_from_f32(b, h, n, acc.shape[-1], _ptr(acc), C.byref(_view_blhd(dst)), _dtype_code(like), _stream()))
        return dst

    return cast(dq, q, lq), cast(dkk, k, lk), cast(dvv, v, lk)


class RingPlan:
    """Which (query shard, K/V block) pairs of a ring have a visible pair at all under a
    `ScoreMod` mask.  With document masks or a sliding window most pairs of a long ring have
    none; `ring_attention(..., plan=plan)` then leaves out their transfers and block launches
    (the reference runs every step, ring.py:104-132).  Made by `make_ring_plan`, collectively,
    once per set of masks: it synchronises the stream once.  The masks of every call that uses
    the plan must be the ones it was made from."""

    def __init__(self, ring: Ring, handle):
        self.ring, self.handle = ring, handle

    def needed(self, q_rank: int, kv_rank: int) -> bool:
        r = lib.ra_ring_plan_need(self.handle, q_rank, kv_rank)
        check(min(r, 0))
        return r == 1

    def matrix(self):
        n = self.ring.size
        return [[self.needed(r, o) for o in range(n)] for r in range(n)]

    def rows(self, q_rank: int, kv_rank: int):
        """Runs [(first, end), ...] of K/V rows of `kv_rank`'s block that travel to `q_rank` (and
        whose dK/dV come back): at most one per half of the block."""
        runs = (C.c_int32 * 4)()
        check(lib.ra_ring_plan_rows(self.handle, q_rank, kv_rank, runs))
        return [(runs[i], runs[i + 1]) for i in (0, 2) if runs[i] < runs[i + 1]]

    def __del__(self):
        if getattr(self, "handle", None):
            lib.ra_ring_plan_destroy(self.handle)
            self.handle = None


def make_ring_plan(q: torch.Tensor, k: torch.Tensor, axis_name, bias_fn, bias_q_kwargs: Optional[dict] = None,
                   bias_kv_kwargs: Optional[dict] = None) -> RingPlan:
    """Plan for ring attention calls with these shard shapes ([b, l, h, d]) and this mask.
    Every rank of the ring must call it (it all-gathers 128-token summaries of the positions,
    segment ids and prefix masks)."""
    if bias_fn is not None and not isinstance(bias_fn, ScoreMod):
        raise ValueError("a plan needs a ScoreMod bias_fn (or None): a callable's bias cannot be summarised")
    ring = resolve_axis(axis_name)
    b, lq, h, dk = q.shape
    mod = _ModArgs(bias_fn, bias_q_kwargs or {}, bias_kv_kwargs or {}, h)
    sh = _shape(b, h, lq, k.shape[1], dk, dk, _dtype_code(q), 1.0)
    handle = C.c_void_p()
    check(lib.ra_ring_plan_create(ring.handle, C.byref(sh), mod.ref(), _stream(), C.byref(handle)))
    return RingPlan(ring, handle)


def reserve(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, axis_name,
            bias_kv_kwargs: Optional[dict] = None, backward: bool = True) -> None:
    """Allocates everything the ring keeps for calls with these shard shapes ([b, l, h, d]) ahead
    of time (`ra_ring_reserve`): afterwards `ring_attention` calls of the same or a smaller shape
    neither allocate inside the library nor synchronise the device.  Every rank must call it."""
    ring = resolve_axis(axis_name)
    b, lq, h, dk = q.shape
    m = None
    if bias_kv_kwargs:
        # only which kv-side arrays exist matters (they travel with K/V); the pointers are not read
        m = RaScoreMod()
        for field, key in (("kv_pos", "kv_positions"), ("kv_seg", "kv_segment_ids"), ("kv_prefix", "kv_prefix_mask")):
            if bias_kv_kwargs.get(key) is not None:
                setattr(m, field, bias_kv_kwargs[key].data_ptr())
    sh = _shape(b, h, lq, k.shape[1], dk, v.shape[3], _dtype_code(q), 1.0)
    check(lib.ra_ring_reserve(ring.handle, C.byref(sh), C.byref(m) if m is not None else None, int(backward)))


class _UsePlan:
    """Applies a plan to a ring handle for the calls inside the `with` block."""

    def __init__(self, ring: Ring, plan: Optional[RingPlan]):
        self.ring, self.plan = ring, plan

    def __enter__(self):
        if self.plan is not None:
            check(lib.ra_ring_use_plan(self.ring.handle, self.plan.handle))

    def __exit__(self, *exc):
        if self.plan is not None:
            check(lib.ra_ring_use_plan(self.ring.handle, None))


class _RingAttention(torch.autograd.Function):
    """The custom-VJP boundary of ring.py:214-243: gradients flow to q, k, v only."""

    @staticmethod
    def forward(ctx, q, k, v, ring, sm_scale, bias_fn, q_kwargs, kv_kwargs, impl, plan):
        q, k, v = _blhd(q), _blhd(k), _blhd(v)
        if ring.size > 1:  # K/V blocks travel as flat messages: slices of a packed projection are copied once
            k, v = k.contiguous(), v.contiguous()
        fused = bias_fn is None or isinstance(bias_fn, ScoreMod)
        check(lib.ra_set_impl(impl))
        fwd = _fused_fwd if fused else _host_fwd
        with _UsePlan(ring, plan if fused else None):
            out, lse = fwd(ring, q, k, v, sm_scale, bias_fn, q_kwargs, kv_kwargs)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.ring, ctx.sm_scale, ctx.bias_fn, ctx.impl, ctx.fused = ring, sm_scale, bias_fn, impl, fused
        ctx.q_kwargs, ctx.kv_kwargs, ctx.plan = q_kwargs, kv_kwargs, plan
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        do = _blhd(do)
        check(lib.ra_set_impl(ctx.impl))
        bwd = _fused_bwd if ctx.fused else _host_bwd
        with _UsePlan(ctx.ring, ctx.plan if ctx.fused else None):
            dq, dk, dv = bwd(ctx.ring, q, k, v, out, lse, do, ctx.sm_scale, ctx.bias_fn, ctx.q_kwargs, ctx.kv_kwargs)
        return dq, dk, dv, None, None, None, None, None, None, None


def ring_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    axis_name,
    bias_fn: Optional[Callable[..., torch.Tensor]] = None,
    bias_q_kwargs: Optional[dict] = None,
    bias_kv_kwargs: Optional[dict] = None,
    sm_scale: Optional[float] = None,
    block_impl: str = "cuda",
    plan: Optional["RingPlan"] = None,
) -> torch.Tensor:
    """Ring attention on this process's shard: the signature of ring.py:246-256, plus `plan`.

    q [b, lq, h, dk], k [b, lk, h, dk], v [b, lk, h, dv] are this rank's blocks of arrays
    sharded on the length axis.  `axis_name` names an axis of the active `Mesh` (or is a
    `Ring`).  `bias_fn(**bias_q_kwargs, **bias_kv_kwargs)` returns an additive bias
    [b, h or 1, lq, lk] for one block; the kv-side kwargs travel round the ring with K/V
    (ring.py:107,120).  A `ScoreMod` bias_fn is evaluated inside the kernels; any other
    callable is honoured through a dense tile per ring step.  `block_impl`: "cuda"
    (default: tcgen05 kernels when the shape fits, fp32 CUDA-core kernels otherwise),
    "tcgen05", "simt"; the reference's "pallas"/"jax" are accepted as "cuda".
    `plan` (from `make_ring_plan`, optional) leaves out the ring steps whose block the mask
    empties; without it every step runs, as in the reference.
    Every rank of the ring must make the same call.
    """
    if sm_scale is None:
        sm_scale = 1 / math.sqrt(q.shape[-1])  # ring.py:287-288
    if bias_q_kwargs is None:
        bias_q_kwargs = {}
    if bias_kv_kwargs is None:
        bias_kv_kwargs = {}
    if block_impl not in _IMPLS:
        raise ValueError(block_impl)  # ring.py:311-312
    _need_cuda(q, k, v)
    if k.shape[2] != q.shape[2] or v.shape[2] != q.shape[2]:
        raise ValueError("q, k and v must have the same number of heads")
    ring = resolve_axis(axis_name)
    return _RingAttention.apply(q, k, v, ring, float(sm_scale), bias_fn, bias_q_kwargs, bias_kv_kwargs,
                                _IMPLS[block_impl], plan)


def ring_self_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    mesh: Optional[Mesh],
    pspec,
    sm_scale: Optional[float] = None,
    causal: bool = False,
    segment_ids: Optional[torch.Tensor] = None,
    positions: Optional[torch.Tensor] = None,
    prefix_mask: Optional[torch.Tensor] = None,
    block_impl: str = "cuda",
    plan: Optional["RingPlan"] = None,
) -> torch.Tensor:
    """Self-attention over this rank's shard: the signature of ring.py:328-340, plus `plan`.

    Arrays are the local shards ([b, l/N, ...]) of arrays partitioned as `pspec` over
    `mesh`; `pspec[1]` names the sequence axis (ring.py:432).  Supports bidirectional,
    segment (block-sparse), causal and prefix-LM masking and their combinations exactly
    as ring.py:386-408; the mask is evaluated inside the kernels from the per-token arrays.
    `mesh=None` with a single process means a ring of one.
    """
    if causal:
        assert positions is not None, "positions are requried for causal attention"
        assert prefix_mask is None, "causal attention does not support prefix_mask"
    if prefix_mask is not None:
        assert positions is not None, "positions are requried for prefixlm attention"
        assert not causal
    needs_mod = causal or segment_ids is not None or prefix_mask is not None
    bias_fn = ScoreMod(causal=causal) if needs_mod else None
    q_kw = {"q_segment_ids": segment_ids, "q_positions": positions, "q_prefix_mask": prefix_mask}
    kv_kw = {"kv_segment_ids": segment_ids, "kv_positions": positions, "kv_prefix_mask": prefix_mask}
    axis = pspec[1]
    ring = mesh.ring(axis) if mesh is not None else resolve_axis(axis)
    return ring_attention(q, k, v, axis_name=ring, sm_scale=sm_scale, bias_fn=bias_fn,
                          bias_q_kwargs=q_kw if needs_mod else None,
                          bias_kv_kwargs=kv_kw if needs_mod else None, block_impl=block_impl, plan=plan)
