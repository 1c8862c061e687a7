"""A numpy stand-in for the few array-library names the reference's source imports.

The reference package is pure Python on top of an array library that is not installed
here.  To obtain golden vectors from the reference's OWN code (rather than from a
re-derivation), ``make_golden.py`` installs this module under the names the
reference imports and then executes the reference's files unmodified.  Only what
those files touch is provided:

* array functions (thin wrappers over numpy, bfloat16 through ``ml_dtypes``),
* ``lax.scan`` / ``vmap`` as Python loops,
* ``custom_vjp`` as an object that runs the registered forward rule, records the
  residuals on a tape, and lets the generator call the registered backward rule,
* ``pallas_call`` as a grid interpreter: for every grid point it slices each operand
  by its block spec, hands numpy views to the kernel body as "refs", and keeps
  scratch buffers alive across grid points -- the semantics of the reference's
  interpret mode.

Automatic differentiation is NOT provided; gradients come only from the
reference's hand-written backward rule.  This file is used by the fixture generator
only and never at test or run time.
"""
from __future__ import annotations

import sys
import types

import ml_dtypes
import numpy as np


class Arr(np.ndarray):
    """ndarray with the functional ``x.at[idx].set(v)`` update."""

    @property
    def at(self):
        return _At(self)


class _At:
    def __init__(self, a):
        self.a = a

    def __getitem__(self, idx):
        return _AtIdx(self.a, idx)


class _AtIdx:
    def __init__(self, a, idx):
        self.a, self.idx = a, idx

    def set(self, v):
        out = np.array(self.a).view(Arr)
        out[self.idx] = v
        return out


def _wrap(x):
    if isinstance(x, np.ndarray):
        return x.view(Arr)
    if isinstance(x, (np.generic,)):
        return np.asarray(x).view(Arr)
    return x


def _f(fn):
    def inner(*a, **k):
        return _wrap(fn(*a, **k))
    inner.__name__ = getattr(fn, "__name__", "fn")
    return inner


TAPE = []          # (op, args, residuals) for every custom_vjp call, newest last
_GRID_POS = [()]   # current grid index for program_id


def _to_f32_if_bf16(x):
    x = np.asarray(x)
    return x.astype(np.float32) if x.dtype == ml_dtypes.bfloat16 else x


def _matmul(a, b, precision=None, preferred_element_type=None):
    r = np.matmul(_to_f32_if_bf16(a), _to_f32_if_bf16(b))
    if preferred_element_type is not None:
        r = r.astype(preferred_element_type)
    return _wrap(r)


def _where(c, a, b):
    return _wrap(np.where(c, a, b))


def _pad(x, pads, constant_values=0, mode="constant"):
    if mode == "constant":
        return _wrap(np.pad(x, pads, mode="constant", constant_values=constant_values))
    return _wrap(np.pad(x, pads, mode=mode))


def _repeat(x, n, axis=None, total_repeat_length=None):
    return _wrap(np.repeat(x, n, axis=axis))


def _dtype(d):
    if isinstance(d, str) and d in ("bfloat16", "bf16"):
        return np.dtype(ml_dtypes.bfloat16)
    return np.dtype(d)


def _tree_stack(items):
    first = items[0]
    if isinstance(first, (tuple, list)):
        return type(first)(_tree_stack([it[i] for it in items]) for i in range(len(first)))
    return _wrap(np.stack([np.asarray(it) for it in items]))


def _tree_index(tree, i):
    if isinstance(tree, (tuple, list)):
        return type(tree)(_tree_index(t, i) for t in tree)
    return _wrap(np.asarray(tree)[i])


def _scan(f, init, xs):
    n = len(np.asarray(xs[0] if isinstance(xs, (tuple, list)) else xs))
    carry, ys = init, []
    for i in range(n):
        carry, y = f(carry, _tree_index(xs, i))
        ys.append(y)
    return carry, _tree_stack(ys)


def _vmap(fn, in_axes=0):
    def mapped(*args):
        n = len(np.asarray(args[0]))
        return _tree_stack([fn(*[_tree_index(a, i) for a in args]) for i in range(n)])
    return mapped


class CustomVJP:
    def __init__(self, fun):
        self.fun = fun
        self.fwd = self.bwd = None

    def defvjp(self, fwd, bwd):
        self.fwd, self.bwd = fwd, bwd

    def __call__(self, *args):
        if self.fwd is None:
            return self.fun(*args)
        out, res = self.fwd(*args)
        TAPE.append((self, args, res))
        return out


class ShapeDtypeStruct:
    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), np.dtype(dtype)


class BlockSpec:
    def __init__(self, block_shape, index_map):
        self.block_shape, self.index_map = tuple(block_shape), index_map

    def view(self, arr, pos):
        idx = self.index_map(*pos)
        sl = tuple(slice(int(i) * s, (int(i) + 1) * s) for i, s in zip(idx, self.block_shape))
        return arr[sl]


class GridSpec:
    def __init__(self, num_scalar_prefetch=0, grid=(), in_specs=(), out_specs=(), scratch_shapes=()):
        self.grid, self.in_specs, self.out_specs = tuple(grid), list(in_specs), list(out_specs)
        self.scratch_shapes = list(scratch_shapes)


class VMEM:
    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), np.dtype(dtype)


def pallas_call(kernel, out_shape=None, grid_spec=None, compiler_params=None, name=None, interpret=True):
    def run(*inputs):
        ins = [np.asarray(x) for x in inputs]
        outs = [np.zeros(s.shape, s.dtype) for s in out_shape]
        scratch = [np.zeros(s.shape, s.dtype) for s in grid_spec.scratch_shapes]
        for pos in np.ndindex(*grid_spec.grid):
            _GRID_POS[0] = pos
            refs = [spec.view(a, pos).view(Arr) for spec, a in zip(grid_spec.in_specs, ins)]
            refs += [spec.view(a, pos).view(Arr) for spec, a in zip(grid_spec.out_specs, outs)]
            refs += [s.view(Arr) for s in scratch]
            kernel(*refs)
        return [o.view(Arr) for o in outs]
    return run


def install():
    """Register the stand-in under the module names the reference imports."""
    jax = types.ModuleType("jax")
    jnp = types.ModuleType("jax.numpy")
    lax = types.ModuleType("jax.lax")
    nn = types.ModuleType("jax.nn")
    core = types.ModuleType("jax.core")
    errors = types.ModuleType("jax.errors")
    adc = types.ModuleType("jax.ad_checkpoint")
    exp = types.ModuleType("jax.experimental")
    pl = types.ModuleType("jax.experimental.pallas")
    pltpu = types.ModuleType("jax.experimental.pallas.tpu")

    for nm in ("sum", "exp", "sqrt", "zeros", "ones", "full", "arange", "eye", "tril", "minimum",
               "maximum", "broadcast_to", "concatenate", "flip", "zeros_like", "ones_like",
               "diff", "cumsum", "asarray", "array"):
        setattr(jnp, nm, _f(getattr(np, nm)))
    jnp.matmul, jnp.where, jnp.pad, jnp.repeat, jnp.dtype = _matmul, _where, _pad, _repeat, _dtype
    jnp.float32, jnp.int32, jnp.integer = np.float32, np.int32, np.integer
    jnp.bfloat16 = ml_dtypes.bfloat16
    jnp.issubdtype = np.issubdtype
    jnp.ndarray = np.ndarray

    class Precision:
        DEFAULT = "default"
        HIGHEST = "highest"

    lax.Precision = Precision
    lax.rsqrt = lambda x: _wrap((1.0 / np.sqrt(x)).astype(np.asarray(x).dtype))
    lax.scan = _scan
    lax.slice = lambda x, lo, hi: _wrap(np.asarray(x)[tuple(slice(a, b) for a, b in zip(lo, hi))])
    nn.sigmoid = lambda x: _wrap((1.0 / (1.0 + np.exp(-np.asarray(x)))).astype(np.asarray(x).dtype))

    class Tracer:  # never instantiated: nothing is traced here
        pass

    core.Tracer = Tracer
    errors.ConcretizationTypeError = type("ConcretizationTypeError", (TypeError,), {})
    adc.checkpoint_name = lambda x, name: x

    jax.numpy, jax.lax, jax.nn, jax.core, jax.errors = jnp, lax, nn, core, errors
    jax.ad_checkpoint, jax.experimental = adc, exp
    jax.Array = np.ndarray
    jax.custom_vjp = CustomVJP
    jax.ShapeDtypeStruct = ShapeDtypeStruct
    jax.default_backend = lambda: "cpu"
    jax.vmap = _vmap
    exp.pallas = pl
    pl.tpu = pltpu
    pl.BlockSpec, pl.pallas_call = BlockSpec, pallas_call
    pl.program_id = lambda axis: _GRID_POS[0][axis]
    pltpu.CompilerParams = lambda **k: None
    pltpu.PrefetchScalarGridSpec = GridSpec
    pltpu.VMEM = VMEM

    sys.modules.update({
        "jax": jax, "jax.numpy": jnp, "jax.lax": lax, "jax.nn": nn, "jax.core": core,
        "jax.errors": errors, "jax.ad_checkpoint": adc, "jax.experimental": exp,
        "jax.experimental.pallas": pl, "jax.experimental.pallas.tpu": pltpu,
    })
    return jax
