"""chunk_gdn2 / gdn2_decode_step on B200: the reference's public operators, same names,
keyword arguments, shapes and error behaviour, running hand-written CUDA kernels through
the C-ABI library.

Mirrors ``src/deltanet_tpu/gdn2.py`` of the reference: ``chunk_gdn2`` (1772-2286) and
``gdn2_decode_step`` (2289-2490).  Tensors are torch CUDA tensors; torch supplies device
memory, streams and the autograd hook that plays the role of the reference's custom VJP
(1446-1769).  All arithmetic on the path is in the CUDA library: the wrapper validates,
describes layouts (gates are passed un-broadcast, lengths un-padded), and allocates.

Deliberate supersets of the reference: ``chunk_size`` may be 64 or 128 and K, V may be
64 or 128 (the reference accepts only 128/128/128, gdn2.py:1869-1870,1897-1898).
``fallback_scan`` is accepted and ignored: there is one implementation.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Union

import numpy as np
import torch

from . import _lib as L

_DT = {torch.float32: L.DN_F32, torch.bfloat16: L.DN_BF16}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _precision_code(precision) -> int:
    if precision is None or not isinstance(precision, str):
        raise ValueError(f"precision must be a string ('bf16' or 'fp32'), got {precision!r}.")
    p = precision.lower()
    if p in ("bf16", "bfloat16"):
        return L.DN_PREC_BF16
    if p in ("fp32", "float32"):
        return L.DN_PREC_FP32
    raise ValueError(f"Invalid precision '{precision}'; must be 'bf16' or 'fp32'.")


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("deltanet_b200 runs on CUDA tensors only; there is no CPU path.")


def _common_dtype(ts: Sequence[torch.Tensor]) -> torch.dtype:
    d = ts[0].dtype
    if d in _DT and all(t.dtype == d for t in ts):
        return d
    return torch.float32


def _gate_layout(x: torch.Tensor, width: int):
    """(heads, cols) of a gate given as (B,L,H) or (B,L,H,1|width)."""
    return (x.shape[2], 1) if x.dim() == 3 else (x.shape[2], x.shape[3])


# --------------------------------------------------------------------------------------------
class _ChunkOp(torch.autograd.Function):
    """The differentiable operator boundary (reference: gdn2.py:1461-1766)."""

    @staticmethod
    def forward(ctx, q, k, v, g, b, w, init_state, seg, shape, want_final, recompute, inference):
        lib = L.lib()
        B, Lq, Hv, V, K = shape.B, shape.L, shape.Hv, shape.V, shape.K
        dev = q.device
        out = torch.empty(B, Lq, Hv, V, dtype=q.dtype, device=dev)
        final = torch.empty(B, Hv, K, V, dtype=torch.float32, device=dev) if want_final else None
        needs_grad = (not inference) and any(ctx.needs_input_grad[:7])
        keep = needs_grad and not recompute
        res_block, res = None, None
        if keep:
            res_block = torch.empty(lib.dn_residual_bytes(shape), dtype=torch.uint8, device=dev)
            res = L.Residuals()
            L.check(lib.dn_residual_carve(shape, res_block.data_ptr(), res), "dn_residual_carve")
        fshape = shape
        if not keep:
            fshape = L.Shape.from_buffer_copy(shape)
            fshape.flags |= L.DN_INFERENCE
        nbytes = lib.dn_scratch_bytes(fshape, 0, 0)
        scratch = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
        L.check(lib.dn_chunk_fwd(fshape, _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(b), _ptr(w), _ptr(seg),
                                 _ptr(init_state), _ptr(out), _ptr(final), res if keep else None,
                                 scratch.data_ptr(), scratch.numel(), _stream()), "dn_chunk_fwd")
        ctx.shape, ctx.inference, ctx.recompute = shape, inference, recompute
        ctx.res_block, ctx.want_final = res_block, want_final
        ctx.has_init = init_state is not None
        ctx.save_for_backward(q, k, v, g, b, w, init_state, seg)
        ctx.set_materialize_grads(False)
        if want_final:
            return out, final
        return out

    @staticmethod
    def backward(ctx, d_out, d_final=None):
        if ctx.inference:
            raise ValueError("chunk_gdn2: differentiation is not supported when is_inference=True; "
                             "set is_inference=False for training.")
        lib = L.lib()
        q, k, v, g, b, w, init_state, seg = ctx.saved_tensors
        shape = ctx.shape
        dev = q.device
        if d_out is None:
            d_out = torch.zeros(shape.B, shape.L, shape.Hv, shape.V, dtype=q.dtype, device=dev)
        d_out = d_out.to(q.dtype).contiguous()
        if d_final is not None:
            d_final = d_final.to(torch.float32).contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dg, db, dw = torch.empty_like(g), torch.empty_like(b), torch.empty_like(w)
        d_init = torch.empty_like(init_state) if ctx.has_init else None
        res = None
        if ctx.res_block is not None:
            res = L.Residuals()
            L.check(lib.dn_residual_carve(shape, ctx.res_block.data_ptr(), res), "dn_residual_carve")
        nbytes = lib.dn_scratch_bytes(shape, 1, 0 if res is not None else 1)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        L.check(lib.dn_chunk_bwd(shape, _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(b), _ptr(w), _ptr(seg),
                                 _ptr(init_state), res, _ptr(d_out), _ptr(d_final),
                                 _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dg), _ptr(db), _ptr(dw), _ptr(d_init),
                                 scratch.data_ptr(), scratch.numel(), _stream()), "dn_chunk_bwd")
        return dq, dk, dv, dg, db, dw, d_init, None, None, None, None, None


def _segments(segment_ids, cu_seqlens, B, Lq, device, first_is_new):
    """Canonical (B,L) int32 ids on the device, or None for a single document."""
    lib = L.lib()
    if segment_ids is not None:
        raw = segment_ids if segment_ids.dim() == 2 else segment_ids[None].expand(B, Lq)
        raw = raw.to(device=device, dtype=torch.int32).contiguous()
    elif cu_seqlens is not None:
        if isinstance(cu_seqlens, torch.Tensor) and cu_seqlens.is_cuda:
            # values on the device are not brought back to the host (no synchronisation), hence not
            # checked, as the reference does not check traced values (gdn2.py:2062-2077)
            cu_dev = cu_seqlens.to(device=device, dtype=torch.int32).contiguous()
        else:
            cu = _validate_cu_seqlens(cu_seqlens, Lq)
            cu_dev = torch.from_numpy(cu.astype(np.int32)).to(device)
        out = torch.empty(B, Lq, dtype=torch.int32, device=device)
        L.check(lib.dn_cu_seqlens_segments(cu_dev.data_ptr(), cu_dev.numel(), _ptr(first_is_new), out.data_ptr(),
                                           B, Lq, _stream()), "dn_cu_seqlens_segments")
        return out, None
    elif first_is_new is not None:
        raw = torch.zeros(B, Lq, dtype=torch.int32, device=device)
    else:
        return None, None
    out = torch.empty_like(raw)
    L.check(lib.dn_canonical_segments(raw.data_ptr(), _ptr(first_is_new), out.data_ptr(), B, Lq, _stream()),
            "dn_canonical_segments")
    return out, raw


def _validate_cu_seqlens(cu_seqlens, Lq):
    """Host-side cu_seqlens checks of the reference (gdn2.py:2041-2061); returns a numpy array."""
    cu = np.asarray(cu_seqlens.detach().cpu() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens)
    if len(cu) == 0 or int(cu[0]) != 0:
        raise ValueError(f"cu_seqlens[0] must be 0, got {int(cu[0]) if len(cu) else 'empty'}.")
    if int(cu[-1]) != Lq:
        raise ValueError(f"cu_seqlens[-1] ({int(cu[-1])}) must equal sequence length ({Lq}).")
    if len(cu) > 1 and np.any(np.diff(cu) <= 0):
        raise ValueError(f"cu_seqlens must be strictly monotonically increasing, got {cu_seqlens}.")
    return cu


def _cap_state(state, tau):
    """stability_guard's Frobenius cap (gdn2.py:2180-2188), in place on a fresh fp32 state."""
    state = state.contiguous()
    n = state.numel() // (state.shape[-2] * state.shape[-1])
    L.check(L.lib().dn_cap_state(state.data_ptr(), n, state.shape[-2], state.shape[-1], float(tau), _stream()),
            "dn_cap_state")
    return state


def chunk_gdn2(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    b: torch.Tensor,
    w: torch.Tensor,
    *,
    segment_ids: Optional[torch.Tensor] = None,
    cu_seqlens=None,
    initial_state: Optional[torch.Tensor] = None,
    initial_state_segment_id: Union[int, torch.Tensor, None] = None,
    output_final_state: bool = False,
    chunk_size: int = 128,
    precision: str = "bf16",
    scale: Optional[float] = None,
    qk_l2norm: bool = False,
    fallback_scan: bool = False,
    is_inference: bool = False,
    fuse_prologue: bool = False,
    recompute_states: bool = False,
    streaming_prefill: bool = False,
    prefill_block_size: int = 4096,
    stability_guard: bool = False,
    stability_tau: float = 1000.0,
    truncate_bwd_dT_bf16: bool = False,
    state_fp32_matmul: bool = False,
    mask_lambda_by_doc: bool = False,
):
    """Chunked GDN-2 recurrence; arguments as the reference's ``chunk_gdn2`` (gdn2.py:1801-1857).

    q, k: (B, L, Hk, K); v: (B, L, Hv, V); g, b: (B, L, H[, 1|K]) with H in {1, Hk, Hv};
    w: (B, L, H[, 1|V]).  Returns ``out`` (B, L, Hv, V) in v's dtype, or ``(out, final_state)``
    with final_state (B, Hv, K, V) float32 when ``output_final_state`` is set.
    ``mask_lambda_by_doc`` is always in effect (the kernels restart the cumulative decay at
    document changes, which is the more precise of the reference's two variants).
    """
    if fuse_prologue and not qk_l2norm:
        raise ValueError(
            "fuse_prologue=True requires qk_l2norm=True because L2-normalization is fused directly "
            "into the kernel prologue.")
    prec = _precision_code(precision)
    if chunk_size not in (64, 128):
        raise ValueError(f"Unsupported chunk_size={chunk_size}; the B200 kernels require chunk_size 64 or 128.")
    if stability_guard and isinstance(stability_tau, (int, float)) and not stability_tau > 0:
        raise ValueError(f"stability_tau must be positive, got {stability_tau}.")
    if streaming_prefill and isinstance(prefill_block_size, int) and not prefill_block_size > 0:
        raise ValueError(f"prefill_block_size must be positive, got {prefill_block_size}.")
    if q.dim() != 4:
        raise ValueError(f"Query tensor q must be 4D (B, L, Hk, K), got shape {tuple(q.shape)}.")
    if k.dim() != 4:
        raise ValueError(f"Key tensor k must be 4D (B, L, Hk, K), got shape {tuple(k.shape)}.")
    if v.dim() != 4:
        raise ValueError(f"Value tensor v must be 4D (B, L, Hv, V), got shape {tuple(v.shape)}.")
    B, Lq, Hk, K = q.shape
    Hv, V = v.shape[2], v.shape[3]
    if tuple(k.shape) != (B, Lq, Hk, K):
        raise ValueError(f"Key tensor k shape {tuple(k.shape)} must match query q shape ({B}, {Lq}, {Hk}, {K}).")
    if v.shape[0] != B or v.shape[1] != Lq:
        raise ValueError(f"Value tensor v shape {tuple(v.shape)} must match query batch and seq dimensions ({B}, {Lq}).")
    if K not in (64, 128) or V not in (64, 128):
        raise ValueError(f"Unsupported head dimensions (K={K}, V={V}); the B200 kernels require K, V in {{64, 128}}.")
    if Hv % Hk != 0:
        raise ValueError(f"Value heads ({Hv}) must be divisible by key heads ({Hk}).")
    for name, x, width, wname in (("g", g, K, "K"), ("b", b, K, "K"), ("w", w, V, "V")):
        if x.dim() not in (3, 4):
            raise ValueError(f"{name} must have rank 3 (B, L, H{name}) or rank 4 (B, L, H{name}, {wname}{name}), "
                             f"got rank {x.dim()} with shape {tuple(x.shape)}.")
        if x.shape[0] != B or x.shape[1] != Lq:
            raise ValueError(f"{name} shape {tuple(x.shape)} must match query batch and seq dimensions ({B}, {Lq}).")
        if x.shape[2] not in (1, Hk, Hv):
            raise ValueError(f"{name} head dimension ({x.shape[2]}) must match key heads ({Hk}) or value heads ({Hv}) or be 1.")
        if x.dim() == 4 and x.shape[3] not in (1, width):
            raise ValueError(f"{name} last dimension ({x.shape[3]}) must be 1 or {wname} ({width}).")
    if segment_ids is not None and cu_seqlens is not None:
        raise ValueError("Cannot pass both segment_ids and cu_seqlens; specify at most one.")
    if cu_seqlens is not None and not (isinstance(cu_seqlens, torch.Tensor) and cu_seqlens.is_cuda):
        _validate_cu_seqlens(cu_seqlens, Lq)
    if segment_ids is not None:
        if segment_ids.dtype.is_floating_point or segment_ids.dtype == torch.bool:
            raise ValueError(f"segment_ids must have integer dtype, got {segment_ids.dtype}.")
        if segment_ids.dim() == 1:
            if segment_ids.shape[0] != Lq:
                raise ValueError(f"1D segment_ids length ({segment_ids.shape[0]}) must match sequence length ({Lq}).")
        elif segment_ids.dim() == 2:
            if tuple(segment_ids.shape) != (B, Lq):
                raise ValueError(f"2D segment_ids shape {tuple(segment_ids.shape)} must match (B={B}, L={Lq}).")
        else:
            raise ValueError(f"segment_ids must be 1D (L,) or 2D (B, L), got rank {segment_ids.dim()} "
                             f"with shape {tuple(segment_ids.shape)}.")
    if initial_state is not None and tuple(initial_state.shape) != (B, Hv, K, V):
        raise ValueError(f"initial_state shape {tuple(initial_state.shape)} must match (B={B}, Hv={Hv}, K={K}, V={V}).")
    if scale is None:
        scale = 1.0 / math.sqrt(K)
    else:
        if isinstance(scale, torch.Tensor) and (scale.requires_grad or scale.numel() != 1):
            raise ValueError("chunk_gdn2: scale must be a concrete Python float or scalar, not a JAX tracer.")
        try:
            scale = float(scale)
        except (TypeError, ValueError) as e:
            raise ValueError(f"chunk_gdn2: scale must be convertible to a concrete float, got {type(scale)}: {e}")
    _require_cuda(q, k, v, g, b, w, initial_state)

    out_dtype = v.dtype
    qkv_dt = _common_dtype((q, k, v))
    gate_dt = _common_dtype((g, b, w))
    q, k, v = (t.to(qkv_dt).contiguous() for t in (q, k, v))
    g, b, w = (t.to(gate_dt).contiguous() for t in (g, b, w))
    if initial_state is not None:
        initial_state = initial_state.to(torch.float32).contiguous()

    first_is_new = None
    if initial_state is not None and initial_state_segment_id is not None:
        isid = torch.as_tensor(initial_state_segment_id, dtype=torch.int32, device=q.device).expand(B)
        if segment_ids is not None:
            s0 = (segment_ids if segment_ids.dim() == 2 else segment_ids[None].expand(B, Lq))[:, 0].to(q.device, torch.int32)
        elif cu_seqlens is not None:
            s0 = torch.zeros(B, dtype=torch.int32, device=q.device)
        else:
            s0 = torch.zeros(B, dtype=torch.int32, device=q.device)
        first_is_new = (s0 != isid).to(torch.int32).contiguous()
    seg, _ = _segments(segment_ids, cu_seqlens, B, Lq, q.device, first_is_new)

    gh, gc = _gate_layout(g, K)
    bh, bc = _gate_layout(b, K)
    wh, wc = _gate_layout(w, V)
    flags = 0
    if qk_l2norm:
        flags |= L.DN_QK_L2NORM
    if fuse_prologue:
        flags |= L.DN_FUSE_PROLOGUE
    if stability_guard:              # the gate clamps (gdn2.py:1972-1974, 141) happen where the kernels load g, b
        flags |= L.DN_STABILITY_GUARD
    if state_fp32_matmul:
        flags |= L.DN_STATE_FP32_MM
    if truncate_bwd_dT_bf16:
        flags |= L.DN_TRUNC_DT_BF16

    def make_shape(length, has_init):
        return L.Shape(B=B, L=length, Hk=Hk, Hv=Hv, K=K, V=V, chunk=chunk_size, g_heads=gh, g_cols=gc,
                       b_heads=bh, b_cols=bc, w_heads=wh, w_cols=wc, qkv_dtype=_DT[qkv_dt],
                       gate_dtype=_DT[gate_dt], precision=prec,
                       flags=flags | (L.DN_HAS_INIT if has_init else 0), scale=scale)

    if is_inference and streaming_prefill and Lq > prefill_block_size:
        if prefill_block_size % chunk_size != 0:
            raise ValueError(f"prefill_block_size ({prefill_block_size}) must be a multiple of chunk_size ({chunk_size}).")
        if seg is None:
            seg = torch.zeros(B, Lq, dtype=torch.int32, device=q.device)
        outs, state = [], initial_state
        for sb in range(0, Lq, prefill_block_size):
            eb = min(sb + prefill_block_size, Lq)
            seg_b = seg[:, sb:eb] if sb == 0 else seg[:, sb:eb] - seg[:, sb - 1:sb]
            o_b, state = _ChunkOp.apply(
                q[:, sb:eb].contiguous(), k[:, sb:eb].contiguous(), v[:, sb:eb].contiguous(),
                g[:, sb:eb].contiguous(), b[:, sb:eb].contiguous(), w[:, sb:eb].contiguous(),
                state, seg_b.contiguous(), make_shape(eb - sb, state is not None), True, False, True)
            if stability_guard:
                state = _cap_state(state, stability_tau)
            outs.append(o_b)
        out = torch.cat(outs, dim=1).to(out_dtype)
        return (out, state) if output_final_state else out

    res = _ChunkOp.apply(q, k, v, g, b, w, initial_state, seg, make_shape(Lq, initial_state is not None),
                         bool(output_final_state), bool(recompute_states), bool(is_inference))
    if output_final_state:
        out, final = res
        if stability_guard and is_inference:
            final = _cap_state(final, stability_tau)
        return out.to(out_dtype), final
    return res.to(out_dtype)


# --------------------------------------------------------------------------------------------
def _torch_dtype(d) -> torch.dtype:
    if d is None:
        return torch.float32
    if isinstance(d, torch.dtype):
        return d
    name = str(d).lower()
    if name in ("bfloat16", "bf16"):
        return torch.bfloat16
    if name in ("float32", "fp32"):
        return torch.float32
    raise ValueError(f"Unsupported state_dtype {d!r}; use 'float32' or 'bfloat16'.")


def gdn2_decode_step(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    b: torch.Tensor,
    w: torch.Tensor,
    state: torch.Tensor,
    *,
    reset=None,
    scale: Optional[float] = None,
    qk_l2norm: bool = False,
    state_dtype=None,
    stability_guard: bool = False,
    stability_tau: float = 1000.0,
    out_state: Optional[torch.Tensor] = None,
):
    """Single-token GDN-2 update; arguments as the reference's ``gdn2_decode_step`` (gdn2.py:2305-2334).

    Returns ``(output, new_state)``.  ``out_state`` (not in the reference) lets a caller supply
    the buffer the new state is written to; passing ``state`` itself updates it in place when
    the dtypes match.
    """
    if stability_guard and isinstance(stability_tau, (int, float)) and not stability_tau > 0:
        raise ValueError(f"stability_tau must be positive, got {stability_tau}.")
    nd = q.dim()
    if nd not in (3, 4):
        raise ValueError(f"Query q must have rank 3 (B, Hk, K) or rank 4 (B, 1, Hk, K), got shape {tuple(q.shape)}.")
    if k.dim() != nd:
        raise ValueError(f"Key k rank ({k.dim()}) must match query rank ({nd}).")
    if v.dim() != nd:
        raise ValueError(f"Value v rank ({v.dim()}) must match query rank ({nd}).")
    if nd == 4:
        if q.shape[1] != 1 or k.shape[1] != 1 or v.shape[1] != 1:
            raise ValueError(f"Decode step sequence dimension must be 1, got q={tuple(q.shape)}, k={tuple(k.shape)}, v={tuple(v.shape)}.")
        q, k, v = q[:, 0], k[:, 0], v[:, 0]
        g = g[:, 0] if g.dim() in (3, 4) and g.shape[1] == 1 else g
        b = b[:, 0] if b.dim() in (3, 4) and b.shape[1] == 1 else b
        w = w[:, 0] if w.dim() in (3, 4) and w.shape[1] == 1 else w
    B, Hk, K = q.shape
    if v.dim() != 3 or v.shape[0] != B:
        raise ValueError(f"Value tensor v batch dimension ({v.shape[0]}) must match query batch dimension ({B}).")
    Hv, V = v.shape[1], v.shape[2]

    def strip(x):
        if x.dim() in (3, 4) and x.shape[0] == B and x.shape[1] == 1 and x.shape[2] in (1, Hk, Hv):
            return x[:, 0]
        return x

    g, b, w = strip(g), strip(b), strip(w)
    if tuple(k.shape) != (B, Hk, K):
        raise ValueError(f"Key tensor k shape {tuple(k.shape)} must match query q shape ({B}, {Hk}, {K}).")
    if K not in (64, 128) or V not in (64, 128):
        raise ValueError(f"Unsupported head dimensions (K={K}, V={V}); requires K, V in {{64, 128}}.")
    if Hv % Hk != 0:
        raise ValueError(f"Value heads ({Hv}) must be divisible by key heads ({Hk}).")
    if tuple(state.shape) != (B, Hv, K, V):
        raise ValueError(f"state shape {tuple(state.shape)} must match ({B}, {Hv}, {K}, {V}).")
    for name, x, width in (("g", g, K), ("b", b, K), ("w", w, V)):
        if x.dim() not in (2, 3) or x.shape[0] != B or x.shape[1] not in (1, Hk, Hv) or \
                (x.dim() == 3 and x.shape[2] not in (1, width)):
            raise ValueError(f"{name} shape {tuple(x.shape)} invalid for batch={B}, Hk={Hk}, Hv={Hv}, "
                             f"{'V' if name == 'w' else 'K'}={width}.")
    tgt = _torch_dtype(state_dtype)
    reset_t, reset_per_head = None, False
    if reset is not None:
        reset_t = torch.as_tensor(reset, device=q.device)
        if reset_t.dim() > 0 and reset_t.shape[0] != B:
            raise ValueError(f"reset batch dimension ({reset_t.shape[0]}) must match input batch dimension ({B}).")
        if reset_t.dim() > 4:
            raise ValueError(f"reset ndim ({reset_t.dim()}) cannot exceed 4.")
        # the reference broadcasts reset over (B,Hv,K,V) (gdn2.py:2404-2410): one flag per sequence, or
        # one per sequence and value head
        if reset_t.dim() == 0:
            reset_t = reset_t.expand(B)
        else:
            while reset_t.dim() > 2 and reset_t.shape[-1] == 1:
                reset_t = reset_t[..., 0]
            if reset_t.dim() == 2 and reset_t.shape[1] == 1:
                reset_t = reset_t[:, 0]
            if reset_t.dim() == 2 and reset_t.shape[1] == v.shape[-2]:
                reset_per_head = True
            elif reset_t.dim() != 1:
                raise ValueError(f"reset shape {tuple(torch.as_tensor(reset).shape)} must broadcast over (B, Hv, 1, 1); "
                                 "per-element resets inside a (K, V) state are not supported.")
        reset_t = reset_t.to(torch.uint8).contiguous()
    _require_cuda(q, k, v, g, b, w, state)
    if scale is None:
        scale = 1.0 / math.sqrt(K)
    out_dtype = v.dtype
    qkv_dt = _common_dtype((q, k, v))
    gate_dt = _common_dtype((g, b, w))
    q, k, v = (t.to(qkv_dt).contiguous() for t in (q, k, v))
    g, b, w = (t.to(gate_dt).contiguous() for t in (g, b, w))
    if state.dtype not in _DT:
        state = state.to(torch.float32)
    state = state.contiguous()
    lay = lambda x: (x.shape[1], 1) if x.dim() == 2 else (x.shape[1], x.shape[2])
    (gh, gc), (bh, bc), (wh, wc) = lay(g), lay(b), lay(w)
    flags = (L.DN_QK_L2NORM if qk_l2norm else 0) | (L.DN_STABILITY_GUARD if stability_guard else 0) | \
        (L.DN_RESET_PER_HEAD if reset_per_head else 0)
    if out_state is None:
        out_state = torch.empty(B, Hv, K, V, dtype=tgt, device=q.device)
    elif out_state.dtype != tgt or tuple(out_state.shape) != (B, Hv, K, V) or not out_state.is_contiguous():
        raise ValueError("out_state must be a contiguous (B, Hv, K, V) tensor of the target state dtype.")
    o = torch.empty(B, Hv, V, dtype=qkv_dt, device=q.device)
    ds = L.DecodeShape(B=B, Hk=Hk, Hv=Hv, K=K, V=V, g_heads=gh, g_cols=gc, b_heads=bh, b_cols=bc,
                       w_heads=wh, w_cols=wc, qkv_dtype=_DT[qkv_dt], gate_dtype=_DT[gate_dt],
                       state_in_dtype=_DT[state.dtype], state_out_dtype=_DT[tgt], flags=flags,
                       scale=float(scale), stability_tau=float(stability_tau))
    L.check(L.lib().dn_decode_step(ds, _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(b), _ptr(w), _ptr(state),
                                   _ptr(reset_t), _ptr(o), _ptr(out_state), _stream()), "dn_decode_step")
    o = o.to(out_dtype)
    if nd == 4:
        o = o[:, None]
    return o, out_state
