"""A NumPy stand-in for the few JAX names the reference's ring.py touches, so that the
reference's own Python (ring_attention/ring.py of jondeaton/ring-attention-jax-pallas) can run
on this machine, where JAX cannot be installed.  Test infrastructure only: it is used by
make_reference_golden.py and by tests/test_reference_run.py, never by the product.

What it provides, and nothing more:

* `jax.numpy`: NumPy, with arrays whose in-place operators return new arrays (JAX arrays are
  immutable, and ring.py writes `mask &= ...` on a 0-d array and `dq += dq_` on carried state);
* `jax.lax.scan` as a Python loop, `jax.lax.psum` / `jax.lax.ppermute` over VIRTUAL ranks:
  every rank is a thread of this process, collectives meet at a barrier and hand pytrees over;
* `jax.custom_vjp`: calling the decorated function runs its forward rule and records the
  residuals on the calling rank's tape; `vjp_of_last_call(cotangent)` runs its backward rule;
* `jax.experimental.shard_map.shard_map`, `jax.sharding.PartitionSpec` / `Mesh`: split the
  arguments along the named axis, run one thread per shard, concatenate the results;
* `jax.experimental.pallas`: an interpreter for the calls ring_kernel.py makes (`pallas_call`
  over a grid with `BlockSpec` blocks, `program_id`, `dslice`, `load`, `dot`, `atomic_add`,
  `cdiv`; `lax.fori_loop`; `ShapeDtypeStruct`): every grid point runs the kernel function on
  views of the operands, one after the other, which is what Pallas' own interpret mode does;
* a placeholder `jaxtyping` so that the imports succeed.

`install()` puts these modules into `sys.modules`; import the reference after it.
"""
from __future__ import annotations

import inspect
import sys
import threading
import types

import numpy as np


# ----------------------------------------------------------------------------- arrays
class FArray(np.ndarray):
    """ndarray whose augmented assignments build a new array (functional, like a JAX array)."""

    def __iadd__(self, other):
        return self + other

    def __isub__(self, other):
        return self - other

    def __imul__(self, other):
        return self * other

    def __itruediv__(self, other):
        return self / other

    def __iand__(self, other):
        return self & other

    def __ior__(self, other):
        return self | other


def _f(x):
    return np.asarray(x).view(FArray)


class _NumpyModule(types.ModuleType):
    """`jax.numpy`: NumPy functions whose array results come back as FArray."""

    def __getattr__(self, name):
        attr = getattr(np, name)
        if not callable(attr) or isinstance(attr, type):
            return attr

        def call(*args, **kwargs):
            out = attr(*args, **kwargs)
            return _f(out) if isinstance(out, np.ndarray) else out

        call.__name__ = name
        return call


# ----------------------------------------------------------------------------- virtual ranks
class _Spmd:
    """N threads that stand for N devices of one mesh axis."""

    def __init__(self, n: int, axis_name: str):
        self.n, self.axis_name = n, axis_name
        self.barrier = threading.Barrier(n)
        self.mailbox = [None] * n
        self.tapes = [[] for _ in range(n)]  # per rank: custom_vjp calls in order


_local = threading.local()


def _ctx() -> _Spmd:
    ctx = getattr(_local, "ctx", None)
    if ctx is None:
        raise RuntimeError("collective outside an SPMD region of the stand-in")
    return ctx


def _rank() -> int:
    return _local.rank


def run_spmd(ctx: _Spmd, fn, per_rank_args):
    """Runs fn(*per_rank_args[r]) on rank r for every rank at once; returns the list of results."""
    results, errors = [None] * ctx.n, [None] * ctx.n

    def body(r):
        _local.ctx, _local.rank = ctx, r
        try:
            results[r] = fn(*per_rank_args[r])
        except BaseException as e:  # noqa: BLE001
            errors[r] = e
            ctx.barrier.abort()

    threads = [threading.Thread(target=body, args=(r,)) for r in range(ctx.n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for e in errors:
        if e is not None and not isinstance(e, threading.BrokenBarrierError):
            raise e
    for e in errors:
        if e is not None:
            raise e
    return results


def _tree_map(f, tree):
    if isinstance(tree, dict):
        return {k: _tree_map(f, v) for k, v in tree.items()}
    if isinstance(tree, (list, tuple)):
        return type(tree)(_tree_map(f, v) for v in tree)
    return None if tree is None else f(tree)


def _psum(x, axis_name):
    ctx = _ctx()
    assert axis_name == ctx.axis_name, (axis_name, ctx.axis_name)
    ctx.mailbox[_rank()] = x
    ctx.barrier.wait()
    total = sum(ctx.mailbox[1:], ctx.mailbox[0])
    ctx.barrier.wait()
    return total


def _ppermute(x, axis_name, perm):
    ctx = _ctx()
    assert axis_name == ctx.axis_name, (axis_name, ctx.axis_name)
    dst = dict(perm)[_rank()]
    ctx.mailbox[dst] = _tree_map(lambda a: _f(np.array(a, copy=True)), x)
    ctx.barrier.wait()
    got = ctx.mailbox[_rank()]
    ctx.barrier.wait()
    return got


def _scan(f, init, xs=None, length=None):
    n = len(xs) if xs is not None else length
    carry = init
    for i in range(n):
        carry, _ = f(carry, None if xs is None else xs[i])
    return carry, None


# ----------------------------------------------------------------------------- custom_vjp
class _CustomVjp:
    def __init__(self, fun, nondiff_argnums=()):
        self.fun, self.nondiff = fun, tuple(nondiff_argnums)
        self.sig = inspect.signature(fun)
        self.fwd = self.bwd = None

    def defvjp(self, fwd, bwd):
        self.fwd, self.bwd = fwd, bwd

    def __call__(self, *args, **kwargs):
        bound = self.sig.bind(*args, **kwargs)
        bound.apply_defaults()
        ordered = list(bound.arguments.values())
        out, residuals = self.fwd(*ordered)
        tape = getattr(_local, "ctx", None)
        if tape is not None:
            tape.tapes[_rank()].append((self, [ordered[i] for i in self.nondiff], residuals))
        return out


def vjp_of_last_call(cotangent):
    """Backward rule of the calling rank's most recent custom_vjp call (collective)."""
    fn, nondiff_args, residuals = _ctx().tapes[_rank()][-1]
    return fn.bwd(*nondiff_args, residuals, cotangent)


def residuals_of_last_call():
    return _ctx().tapes[_rank()][-1][2]


# ----------------------------------------------------------------------------- shard_map
LAST_CTX = None  # the SPMD region of the most recent shard_map call (its tapes stay readable)


class PartitionSpec(tuple):
    def __new__(cls, *names):
        return super().__new__(cls, names)


class Mesh:
    def __init__(self, n: int, axis_names=("dp", "sp")):
        self.shape = {axis_names[0]: 1, axis_names[1]: n}
        self.axis_names = tuple(axis_names)


def _split(tree, spec, n):
    axis = [i for i, name in enumerate(spec) if name is not None]
    assert len(axis) == 1, spec
    return [_tree_map(lambda a: _f(np.array_split(np.asarray(a), n, axis=axis[0])[r]), tree) for r in range(n)]


def shard_map(fn, mesh, in_specs, out_specs, check_rep=True):
    del check_rep
    names = [name for name in out_specs if name is not None]
    n, axis_name = mesh.shape[names[0]], names[0]

    def run(*args):
        ctx = _Spmd(n, axis_name)
        shards = [_split(a, s, n) for a, s in zip(args, in_specs)]
        outs = run_spmd(ctx, fn, [[s[r] for s in shards] for r in range(n)])
        axis = [i for i, name in enumerate(out_specs) if name is not None][0]
        global LAST_CTX
        LAST_CTX = ctx
        if isinstance(outs[0], tuple):
            return tuple(_f(np.concatenate([o[i] for o in outs], axis=axis)) for i in range(len(outs[0])))
        return _f(np.concatenate(outs, axis=axis))

    return run


# ----------------------------------------------------------------------------- pallas
class _Ref:
    """A block of an operand as the kernel sees it: `ref[...]`, `ref.shape`, `pl.load(ref, idx)`."""

    def __init__(self, view):
        self.view = view

    shape = property(lambda self: self.view.shape)
    dtype = property(lambda self: self.view.dtype)

    def __getitem__(self, idx):
        return _f(np.array(self.view[idx], copy=True))

    def __setitem__(self, idx, value):
        self.view[idx] = value


class BlockSpec:
    def __init__(self, block_shape, index_map):
        self.block_shape, self.index_map = tuple(block_shape), index_map


class ShapeDtypeStruct:
    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), dtype


_grid_index = threading.local()


def _program_id(axis):
    return _grid_index.value[axis]


def _dslice(start, size=None):
    return slice(0, start) if size is None else slice(start, start + size)


def _block_view(array, spec, index):
    """The block a BlockSpec selects at one grid point.  A block index past the end is clamped
    so that the block stays inside the array, as lax.dynamic_slice (and with it Pallas'
    interpret mode) does."""
    where = spec.index_map(*index)
    idx = []
    for dim, (size, i) in enumerate(zip(spec.block_shape, where)):
        if size is None:  # a squeezed dimension is a block of one row, clamped like the others
            idx.append(min(int(i), array.shape[dim] - 1))  # (a [b, 1, lq, lk] bias serves every head)
        else:
            start = min(int(i) * size, max(array.shape[dim] - size, 0))
            idx.append(slice(start, start + size))
    return array[tuple(idx)]


def _pallas_call(kernel, grid, in_specs, out_specs, out_shape, input_output_aliases=None, **unused):
    single = not isinstance(out_shape, (list, tuple))
    out_shapes = [out_shape] if single else list(out_shape)
    out_specs_l = [out_specs] if single else list(out_specs)

    def run(*args):
        args = [None if a is None else np.asarray(a) for a in args]
        outs = [np.zeros(s.shape, s.dtype) for s in out_shapes]
        present = [a for a in args if a is not None]  # alias indices count the operands that exist
        for src, dst in (input_output_aliases or {}).items():
            outs[dst] = np.array(present[src], dtype=out_shapes[dst].dtype, copy=True)
        for index in np.ndindex(*grid):
            _grid_index.value = index
            refs = [None if a is None else _Ref(_block_view(a, s, index)) for a, s in zip(args, in_specs)]
            refs += [_Ref(_block_view(o, s, index)) for o, s in zip(outs, out_specs_l)]
            kernel(*refs)
        outs = [_f(o) for o in outs]
        return outs[0] if single else outs

    return run


def _fori_loop(lower, upper, body, init):
    carry = init
    for i in range(int(lower), int(upper)):
        carry = body(i, carry)
    return carry


def _atomic_add(ref, idx, value):
    ref.view[idx] += np.asarray(value).astype(ref.view.dtype)


# ----------------------------------------------------------------------------- install
class _Subscript:
    def __getitem__(self, item):
        return self


def install():
    if "jax" in sys.modules and not getattr(sys.modules["jax"], "_numpy_standin", False):
        raise RuntimeError("a real jax is imported: the stand-in is not needed")
    jax = types.ModuleType("jax")
    jax._numpy_standin = True
    jnp = _NumpyModule("jax.numpy")
    lax = types.ModuleType("jax.lax")
    lax.scan, lax.psum, lax.ppermute, lax.fori_loop = _scan, _psum, _ppermute, _fori_loop
    sharding = types.ModuleType("jax.sharding")
    sharding.PartitionSpec, sharding.Mesh = PartitionSpec, Mesh
    experimental = types.ModuleType("jax.experimental")
    sm = types.ModuleType("jax.experimental.shard_map")
    sm.shard_map = shard_map
    pallas = types.ModuleType("jax.experimental.pallas")
    pallas.program_id, pallas.dslice, pallas.ds = _program_id, _dslice, _dslice
    pallas.load = lambda ref, idx: ref[idx]
    pallas.dot = lambda a, b: _f(np.asarray(a) @ np.asarray(b))
    pallas.cdiv = lambda a, b: -(-a // b)
    pallas.atomic_add, pallas.BlockSpec, pallas.pallas_call = _atomic_add, BlockSpec, _pallas_call
    experimental.shard_map, experimental.pallas = sm, pallas
    jax.numpy, jax.lax, jax.sharding, jax.experimental = jnp, lax, sharding, experimental
    jax.custom_vjp = _CustomVjp
    jax.Array = np.ndarray
    jax.ShapeDtypeStruct = ShapeDtypeStruct
    jaxtyping = types.ModuleType("jaxtyping")
    for name in ("Float", "Int", "Bool", "PyTree"):
        setattr(jaxtyping, name, _Subscript())
    jaxtyping.Array = np.ndarray
    sys.modules.update({
        "jax": jax, "jax.numpy": jnp, "jax.lax": lax, "jax.sharding": sharding,
        "jax.experimental": experimental, "jax.experimental.shard_map": sm,
        "jax.experimental.pallas": pallas, "jaxtyping": jaxtyping,
    })
    return jax


def uninstall():
    if not getattr(sys.modules.get("jax"), "_numpy_standin", False):
        return
    for name in ("jax", "jax.numpy", "jax.lax", "jax.sharding", "jax.experimental",
                 "jax.experimental.shard_map", "jax.experimental.pallas", "jaxtyping"):
        sys.modules.pop(name, None)
