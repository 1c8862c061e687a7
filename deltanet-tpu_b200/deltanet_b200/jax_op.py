"""JAX front end: ``chunk_gdn2`` as a ``jax.custom_vjp`` whose forward and backward are XLA FFI custom calls
into this library.

OPTIONAL.  Importing this module needs ``jax`` (with ``jax.ffi``) and the FFI shim
``libdeltanet_b200_ffi.so`` that ``csrc/build_ffi.sh`` builds where jaxlib is installed; the rest of the
package (the torch front end, the C ABI) does not depend on it.  The image this package is developed on
has no jaxlib, so this module is not exercised there.

It mirrors the reference's operator factory (``src/deltanet_tpu/gdn2.py:1446-1477``): one cached
``custom_vjp`` per static configuration -- the same cache key (chunk_size, precision, with_final_state,
has_init_state, fuse_prologue, scale, recompute_states, truncate_bwd_dT_bf16, state_fp32_matmul,
stability_guard) -- whose residuals are the inputs plus ONE opaque residual block, tagged with
``checkpoint_name`` like the reference's prepass outputs (``gdn2.py:1280-1286``) so that a remat policy can
choose to save or drop it.  Workspace is requested from XLA as an extra result of the custom call.
Batch / head sharding composes with ``jax.shard_map`` exactly as in the reference (``README.md:84-99``):
the op has no cross-device dependence along B or H.
"""
from __future__ import annotations

import ctypes
import functools
import math
import os

import jax
import jax.numpy as jnp
import numpy as np
from jax.ad_checkpoint import checkpoint_name

from . import _lib as L

_HERE = os.path.dirname(os.path.abspath(__file__))
_FFI_PATH = os.path.join(_HERE, "libdeltanet_b200_ffi.so")
_registered = False


def _register():
    global _registered
    if _registered:
        return
    if not os.path.exists(_FFI_PATH):
        raise RuntimeError(f"deltanet_b200.jax_op: {_FFI_PATH} is missing; build it with deltanet-tpu_b200/csrc/build_ffi.sh")
    L.lib()                                            # the C-ABI library the shim links against
    shim = ctypes.CDLL(_FFI_PATH)
    for name in ("dn_ffi_chunk_fwd", "dn_ffi_chunk_bwd", "dn_ffi_decode_step"):
        jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(getattr(shim, name)), platform="CUDA")
    _registered = True


def _dt(x):
    return L.DN_BF16 if x.dtype == jnp.bfloat16 else L.DN_F32


def _gate_layout(x):
    return (x.shape[2], 1) if x.ndim == 3 else (x.shape[2], x.shape[3])


def _shape_struct(q, v, g, b, w, chunk, precision, flags, scale):
    (gh, gc), (bh, bc), (wh, wc) = _gate_layout(g), _gate_layout(b), _gate_layout(w)
    B, Lq, Hk, K = q.shape
    return L.Shape(B=B, L=Lq, Hk=Hk, Hv=v.shape[2], K=K, V=v.shape[3], chunk=chunk, g_heads=gh, g_cols=gc, b_heads=bh,
                   b_cols=bc, w_heads=wh, w_cols=wc, qkv_dtype=_dt(q), gate_dtype=_dt(g), precision=precision,
                   flags=flags, scale=scale)


@functools.lru_cache(maxsize=32)
def _get_op(chunk_size, precision, with_final_state, has_init_state, fuse_prologue, scale, recompute_states,
            truncate_bwd_dT_bf16, state_fp32_matmul, stability_guard, qk_l2norm):
    _register()
    lib = L.lib()
    flags = ((L.DN_QK_L2NORM if qk_l2norm else 0) | (L.DN_FUSE_PROLOGUE if fuse_prologue else 0) |
             (L.DN_HAS_INIT if has_init_state else 0) | (L.DN_STABILITY_GUARD if stability_guard else 0) |
             (L.DN_STATE_FP32_MM if state_fp32_matmul else 0) | (L.DN_TRUNC_DT_BF16 if truncate_bwd_dT_bf16 else 0))
    attrs = dict(chunk=np.int64(chunk_size), precision=np.int64(precision), flags=np.int64(flags), scale=np.float32(scale))

    def call_fwd(q, k, v, g, b, w, seg, init, keep):
        s = _shape_struct(q, v, g, b, w, chunk_size, precision, flags | (0 if keep else L.DN_INFERENCE), scale)
        B, Lq, Hk, K = q.shape
        Hv, V = v.shape[2], v.shape[3]
        res_bytes = lib.dn_residual_bytes(s) if keep else 1
        outs = (jax.ShapeDtypeStruct((B, Lq, Hv, V), q.dtype), jax.ShapeDtypeStruct((B, Hv, K, V), jnp.float32),
                jax.ShapeDtypeStruct((res_bytes,), jnp.uint8),
                jax.ShapeDtypeStruct((max(lib.dn_scratch_bytes(s, 0, 0), 256),), jnp.uint8))
        out, final, res, _ = jax.ffi.ffi_call("dn_ffi_chunk_fwd", outs)(q, k, v, g, b, w, seg, init, keep_residuals=keep, **attrs)
        return out, final, res

    def call_bwd(q, k, v, g, b, w, seg, init, res, d_out, d_final):
        s = _shape_struct(q, v, g, b, w, chunk_size, precision, flags, scale)
        sd = lambda x: jax.ShapeDtypeStruct(x.shape, x.dtype)
        outs = (sd(q), sd(k), sd(v), sd(g), sd(b), sd(w), sd(init),
                jax.ShapeDtypeStruct((lib.dn_scratch_bytes(s, 1, 1 if recompute_states else 0),), jnp.uint8))
        r = jax.ffi.ffi_call("dn_ffi_chunk_bwd", outs)(q, k, v, g, b, w, seg, init, res, d_out, d_final,
                                                       recompute_states=recompute_states, **attrs)
        return r[:7]

    @jax.custom_vjp
    def op(q, k, v, g, b, w, seg, init):
        out, final, _ = call_fwd(q, k, v, g, b, w, seg, init, False)
        return (out, final) if with_final_state else out

    def fwd(q, k, v, g, b, w, seg, init):
        keep = not recompute_states
        out, final, res = call_fwd(q, k, v, g, b, w, seg, init, keep)
        res = checkpoint_name(res, "gdn_residuals")      # W, U, M, qe, ke, Lambda_end, T and the chunk states in one block
        return ((out, final) if with_final_state else out), (q, k, v, g, b, w, seg, init, res)

    def bwd(saved, cot):
        q, k, v, g, b, w, seg, init, res = saved
        d_out, d_final = cot if with_final_state else (cot, jnp.zeros((q.shape[0], v.shape[2], q.shape[3], v.shape[3]), jnp.float32))
        dq, dk, dv, dg, db, dw, d_init = call_bwd(q, k, v, g, b, w, seg, init, res, d_out.astype(q.dtype),
                                                  d_final.astype(jnp.float32))
        return dq, dk, dv, dg, db, dw, None, (d_init if has_init_state else jnp.zeros_like(init))

    op.defvjp(fwd, bwd)
    return op


def chunk_gdn2(q, k, v, g, b, w, *, segment_ids=None, initial_state=None, output_final_state=False, chunk_size=128,
               precision="bf16", scale=None, qk_l2norm=False, fuse_prologue=False, recompute_states=False,
               stability_guard=False, truncate_bwd_dT_bf16=False, state_fp32_matmul=False):
    """``chunk_gdn2`` for JAX arrays on a CUDA device; arguments as the reference's (``gdn2.py:1772-1800``).

    Segment ids are canonicalised with jnp integer ops before the custom call (a cumulative count of id
    changes, ``gdn2.py:2087-2094``); everything else happens inside the library.
    """
    if fuse_prologue and not qk_l2norm:
        raise ValueError("fuse_prologue=True requires qk_l2norm=True because L2-normalization is fused directly "
                         "into the kernel prologue.")
    if not isinstance(precision, str) or precision.lower() not in ("bf16", "bfloat16", "fp32", "float32"):
        raise ValueError(f"Invalid precision '{precision}'; must be 'bf16' or 'fp32'.")
    prec = L.DN_PREC_BF16 if precision.lower() in ("bf16", "bfloat16") else L.DN_PREC_FP32
    B, Lq, Hk, K = q.shape
    Hv, V = v.shape[2], v.shape[3]
    if scale is None:
        scale = 1.0 / math.sqrt(K)
    elif isinstance(scale, jax.core.Tracer):
        raise ValueError("chunk_gdn2: scale must be a concrete Python float or scalar, not a JAX tracer.")
    if segment_ids is None:
        seg = jnp.zeros((B, Lq), jnp.int32)
    else:
        raw = jnp.broadcast_to(segment_ids[None], (B, Lq)) if segment_ids.ndim == 1 else segment_ids
        chg = (raw[:, 1:] != raw[:, :-1]).astype(jnp.int32)
        seg = jnp.concatenate([jnp.zeros((B, 1), jnp.int32), jnp.cumsum(chg, axis=1)], axis=1)
    has_init = initial_state is not None
    init = initial_state.astype(jnp.float32) if has_init else jnp.zeros((B, Hv, K, V), jnp.float32)
    op = _get_op(int(chunk_size), prec, bool(output_final_state), has_init, bool(fuse_prologue), float(scale),
                 bool(recompute_states), bool(truncate_bwd_dT_bf16), bool(state_fp32_matmul), bool(stability_guard),
                 bool(qk_l2norm))
    return op(q, k, v, g, b, w, seg, init)
