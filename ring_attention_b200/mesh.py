"""Named mesh axes for one-process-per-GPU programs.

The reference runs under `shard_map` over a `jax.sharding.Mesh` and names the sequence
axis by string (ring_attention/ring.py:249, 422-449; ring_test.py:60-65).  Here every
process already holds its shard, so a `Mesh` only has to map an axis name to the ring
of processes that share it.  `Ring` owns the native handle (`ra_ring_t`).
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import check, lib


class PartitionSpec(tuple):
    """`PartitionSpec("dp", "sp", None)`: axis names per array dimension (ring_test.py:76-80)."""

    def __new__(cls, *names):
        return super().__new__(cls, names)


class Ring:
    """One rank's place in a ring of GPUs: replaces `axis_name` + ppermute (ring.py:41-55)."""

    def __init__(self, rank: int = 0, nranks: int = 1, nccl_id: Optional[bytes] = None):
        if not torch.cuda.is_available():
            raise _lib.RingAttentionError("ring_attention_b200 needs a CUDA device (no CPU fallback)")
        handle = C.c_void_p()
        idbuf = None
        if nranks > 1:
            if nccl_id is None or len(nccl_id) != _lib.RA_UNIQUE_ID_BYTES:
                raise ValueError("nccl_id of 128 bytes is required when nranks > 1")
            idbuf = C.create_string_buffer(nccl_id, _lib.RA_UNIQUE_ID_BYTES)
        check(lib.ra_ring_create(rank, nranks, C.cast(idbuf, C.c_void_p) if idbuf else None, C.byref(handle)))
        self._h = handle
        self.rank, self.size = rank, nranks
        self.device = torch.cuda.current_device()

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(_lib.RA_UNIQUE_ID_BYTES)
        check(lib.ra_ring_unique_id(C.cast(buf, C.c_void_p)))
        return buf.raw

    @classmethod
    def from_ranks(cls, ranks: Sequence[int]) -> "Ring":
        """Collective over the default torch.distributed group: builds the ring made of
        the global ranks `ranks` (every process must call it, with its own group)."""
        import torch.distributed as dist

        me = dist.get_rank() if dist.is_initialized() else 0
        ranks = list(ranks)
        if len(ranks) == 1:
            return cls(0, 1)
        mine = cls.unique_id() if ranks[0] == me else None
        ids = [None] * dist.get_world_size()
        dist.all_gather_object(ids, mine)
        return cls(ranks.index(me), len(ranks), ids[ranks[0]])

    @property
    def handle(self) -> C.c_void_p:
        if self._h is None:
            raise _lib.RingAttentionError("ring handle was destroyed")
        return self._h

    def set_timing(self, on: bool) -> None:
        check(lib.ra_ring_set_timing(self.handle, int(on)))

    def last_timing(self, backward: bool):
        """(total device ms, ms the compute stream waited on transfers) of the last forward / backward call."""
        tot, exp = C.c_float(), C.c_float()
        check(lib.ra_ring_last_timing(self.handle, int(backward), C.byref(tot), C.byref(exp)))
        return tot.value, exp.value

    def last_block_ms(self, backward: bool):
        """(device ms of the block kernels, launches) of the last forward / backward ring call."""
        ms, n = C.c_float(), C.c_int32()
        check(lib.ra_ring_last_block_ms(self.handle, int(backward), C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def last_timeline(self, backward: bool, max_items: int = 64):
        """([(begin, end)] of the block launches, [(begin, end)] of the waits for transfers), in ms
        from the start of the last forward / backward ring call."""
        b, w = (C.c_float * (2 * max_items))(), (C.c_float * (2 * max_items))()
        nb, nw = C.c_int32(), C.c_int32()
        check(lib.ra_ring_last_timeline(self.handle, int(backward), max_items, b, C.byref(nb), w, C.byref(nw)))
        return ([(b[2 * i], b[2 * i + 1]) for i in range(nb.value)], [(w[2 * i], w[2 * i + 1]) for i in range(nw.value)])

    def last_push(self, backward: bool):
        """(bytes this rank pushed to peers, device ms of those copies) in the last forward / backward ring call."""
        nbytes, ms = C.c_double(), C.c_float()
        check(lib.ra_ring_last_push(self.handle, int(backward), C.byref(nbytes), C.byref(ms)))
        return nbytes.value, ms.value

    @property
    def transport(self) -> str:
        """"none" (ring of one), "p2p" (peer copies over CUDA IPC) or "nccl"."""
        return {0: "none", 1: "p2p", 2: "nccl"}[lib.ra_ring_transport(self.handle)]

    def set_wait_ms(self, ms: int) -> None:
        """Bound of one wait for a peer; a wait that runs out aborts the ring (see `aborted`)."""
        check(lib.ra_ring_set_wait_ms(self.handle, int(ms)))

    @property
    def aborted(self) -> bool:
        """True once a wait for a peer has run out: results since then are undefined and the
        ring must be destroyed and created again on every rank."""
        r = lib.ra_ring_aborted(self.handle)
        check(min(r, 0))
        return r == 1

    def destroy(self) -> None:
        if getattr(self, "_h", None) is not None:
            lib.ra_ring_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class Mesh:
    """Axis names over the processes of the default torch.distributed group.

    `Mesh((1, 8), ("dp", "sp"))` mirrors `Mesh(create_device_mesh((1, 8)), ("dp", "sp"))`
    of ring_test.py:60-65: process `r` sits at the row-major coordinate of `r` in `shape`.
    """

    def __init__(self, shape: Sequence[int], axis_names: Sequence[str]):
        import torch.distributed as dist

        self.shape = tuple(int(s) for s in shape)
        self.axis_names = tuple(axis_names)
        if len(self.shape) != len(self.axis_names):
            raise ValueError("shape and axis_names differ in length")
        world = dist.get_world_size() if dist.is_initialized() else 1
        me = dist.get_rank() if dist.is_initialized() else 0
        total = 1
        for s in self.shape:
            total *= s
        if total != world:
            raise ValueError(f"mesh shape {self.shape} needs {total} processes, world has {world}")
        self.coords = self.coords_of(me, self.shape)
        self._rings = {}
        for ax, name in enumerate(self.axis_names):
            self._rings[name] = Ring.from_ranks(self.axis_ranks(me, ax, self.shape))

    @staticmethod
    def coords_of(rank: int, shape: Sequence[int]):
        out = []
        for s in reversed(shape):
            out.append(rank % s)
            rank //= s
        return tuple(reversed(out))

    @staticmethod
    def axis_ranks(rank: int, axis: int, shape: Sequence[int]):
        """Global ranks that differ from `rank` only in mesh coordinate `axis`, in order."""
        coords = list(Mesh.coords_of(rank, shape))
        out = []
        for i in range(shape[axis]):
            coords[axis] = i
            r = 0
            for c, s in zip(coords, shape):
                r = r * s + c
            out.append(r)
        return out

    def ring(self, axis_name: str) -> Ring:
        return self._rings[axis_name]

    def __enter__(self):
        _stack().append(self)
        return self

    def __exit__(self, *exc):
        _stack().pop()


_tls = threading.local()


def _stack():
    if not hasattr(_tls, "stack"):
        _tls.stack = []
    return _tls.stack


_default_ring: Optional[Ring] = None


def resolve_axis(axis_name) -> Ring:
    """Ring for `axis_name`: a Ring passes through; a string is looked up in the active Mesh."""
    global _default_ring
    if isinstance(axis_name, Ring):
        return axis_name
    st = _stack()
    if st:
        return st[-1].ring(axis_name)
    import torch.distributed as dist

    if dist.is_initialized() and dist.get_world_size() > 1:
        raise _lib.RingAttentionError(
            f"axis {axis_name!r}: no Mesh is active; wrap the call in `with Mesh(shape, names):`"
        )
    if _default_ring is None or _default_ring.device != torch.cuda.current_device():
        _default_ring = Ring(0, 1)
    return _default_ring
