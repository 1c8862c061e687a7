"""The steps either side of the recurrence in a Gated DeltaNet layer, on the same C-ABI library.

The reference's layer example (``examples/qwen3_5_layer_parity.py:144-159``) wires a Qwen3.5 linear-attention
layer around ``chunk_gdn``: the projected activations pass a short depthwise causal convolution and SiLU and
are split into q, k, v; the gate pre-activations become ``g = -exp(A_log) * softplus(a + dt_bias)`` and
``beta = sigmoid(b)``; the recurrence's output is normalised per value head and gated,
``weight * rmsnorm(o) * silu(z)``.  These three functions are those steps as CUDA kernels (forward and
backward, differentiable through torch autograd), so that a layer runs
``gdn_qkv_producer -> gdn_gates -> chunk_gdn -> gated_rmsnorm`` without any eager element-wise op in between.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib as L
from .gdn2 import _DT, _ptr, _require_cuda, _stream


def _f32(t):
    return None if t is None else t.detach().to(torch.float32).contiguous()


class _Producer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, mixed, conv_w, conv_b, seg, Hk, Hv, K, V):
        lib = L.lib()
        B, Lq, D = mixed.shape
        W = conv_w.shape[-1]
        mixed = mixed.contiguous()
        w32, b32 = _f32(conv_w.reshape(D, W)), _f32(conv_b)
        q = torch.empty(B, Lq, Hk, K, dtype=mixed.dtype, device=mixed.device)
        k = torch.empty_like(q)
        v = torch.empty(B, Lq, Hv, V, dtype=mixed.dtype, device=mixed.device)
        L.check(lib.dn_gdn_producer_fwd(mixed.data_ptr(), w32.data_ptr(), _ptr(b32), _ptr(seg), B, Lq, Hk, Hv, K, V, W,
                                        _DT[mixed.dtype], q.data_ptr(), k.data_ptr(), v.data_ptr(), _stream()),
                "dn_gdn_producer_fwd")
        ctx.save_for_backward(mixed, w32, b32, seg)
        ctx.dims = (B, Lq, Hk, Hv, K, V, W, D)
        ctx.w_like, ctx.b_like = conv_w, conv_b
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        lib = L.lib()
        mixed, w32, b32, seg = ctx.saved_tensors
        B, Lq, Hk, Hv, K, V, W, D = ctx.dims
        dq, dk, dv = (t.to(mixed.dtype).contiguous() for t in (dq, dk, dv))
        d_mixed = torch.empty_like(mixed)
        dw = torch.empty(D, W, dtype=torch.float32, device=mixed.device)
        db = torch.empty(D, dtype=torch.float32, device=mixed.device) if b32 is not None else None
        n = lib.dn_gdn_producer_scratch_bytes(B, Lq, D, W)
        scratch = torch.empty(n, dtype=torch.uint8, device=mixed.device)
        L.check(lib.dn_gdn_producer_bwd(mixed.data_ptr(), w32.data_ptr(), _ptr(b32), _ptr(seg), B, Lq, Hk, Hv, K, V, W,
                                        _DT[mixed.dtype], dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), d_mixed.data_ptr(),
                                        dw.data_ptr(), _ptr(db), scratch.data_ptr(), n, _stream()), "dn_gdn_producer_bwd")
        dw = dw.reshape(ctx.w_like.shape).to(ctx.w_like.dtype)
        return d_mixed, dw, (None if db is None else db.to(ctx.b_like.dtype)), None, None, None, None, None


def gdn_qkv_producer(mixed_qkv: torch.Tensor, conv_weight: torch.Tensor, conv_bias: Optional[torch.Tensor] = None, *,
                     num_k_heads: int, num_v_heads: int, head_k_dim: int = 128, head_v_dim: int = 128,
                     segment_ids: Optional[torch.Tensor] = None):
    """Depthwise causal convolution + SiLU + split: ``mixed_qkv`` (B, L, 2*Hk*K + Hv*V) -> q, k (B,L,Hk,K), v (B,L,Hv,V).

    ``conv_weight`` is (D, W) or torch's (D, 1, W) with W in {2,3,4}; the last tap multiplies the current
    token.  With ``segment_ids`` (B, L) or (L,), taps do not reach across a document boundary (the packed
    counterpart of left padding each document with zeros).
    """
    if mixed_qkv.dim() != 3:
        raise ValueError(f"mixed_qkv must be (B, L, D), got shape {tuple(mixed_qkv.shape)}.")
    B, Lq, D = mixed_qkv.shape
    if D != 2 * num_k_heads * head_k_dim + num_v_heads * head_v_dim:
        raise ValueError(f"mixed_qkv last dimension ({D}) must equal 2*Hk*K + Hv*V "
                         f"({2 * num_k_heads * head_k_dim + num_v_heads * head_v_dim}).")
    if conv_weight.shape[0] != D or conv_weight.shape[-1] not in (2, 3, 4) or conv_weight.numel() != D * conv_weight.shape[-1]:
        raise ValueError(f"conv_weight shape {tuple(conv_weight.shape)} must be (D, W) or (D, 1, W) with W in {{2,3,4}}.")
    if mixed_qkv.dtype not in _DT:
        raise ValueError(f"mixed_qkv dtype {mixed_qkv.dtype} must be float32 or bfloat16.")
    _require_cuda(mixed_qkv, conv_weight, conv_bias)
    seg = None
    if segment_ids is not None:
        raw = segment_ids if segment_ids.dim() == 2 else segment_ids[None].expand(B, Lq)
        raw = raw.to(device=mixed_qkv.device, dtype=torch.int32).contiguous()
        seg = torch.empty_like(raw)
        L.check(L.lib().dn_canonical_segments(raw.data_ptr(), None, seg.data_ptr(), B, Lq, _stream()), "dn_canonical_segments")
    return _Producer.apply(mixed_qkv, conv_weight, conv_bias, seg, num_k_heads, num_v_heads, head_k_dim, head_v_dim)


class _Gates(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, A_log, dt_bias):
        lib = L.lib()
        B, Lq, Hv = a.shape
        dt = a.dtype if a.dtype in _DT and a.dtype == b.dtype else torch.float32
        a_, b_ = a.to(dt).contiguous(), b.to(dt).contiguous()
        A32, d32 = _f32(A_log), _f32(dt_bias)
        g = torch.empty(B, Lq, Hv, dtype=torch.float32, device=a.device)
        beta = torch.empty_like(g)
        L.check(lib.dn_gdn_gates_fwd(a_.data_ptr(), b_.data_ptr(), A32.data_ptr(), d32.data_ptr(), B, Lq, Hv, _DT[dt],
                                     g.data_ptr(), beta.data_ptr(), _stream()), "dn_gdn_gates_fwd")
        ctx.save_for_backward(a_, b_, A32, d32)
        ctx.like = (a.dtype, b.dtype, A_log.dtype, dt_bias.dtype)
        ctx.set_materialize_grads(False)
        return g, beta

    @staticmethod
    def backward(ctx, dg, dbeta):
        lib = L.lib()
        a_, b_, A32, d32 = ctx.saved_tensors
        B, Lq, Hv = a_.shape
        z = lambda t: torch.zeros(B, Lq, Hv, dtype=torch.float32, device=a_.device) if t is None else t.to(torch.float32).contiguous()
        dg, dbeta = z(dg), z(dbeta)
        da, db = torch.empty_like(a_), torch.empty_like(b_)
        dA, dD = torch.empty_like(A32), torch.empty_like(d32)
        L.check(lib.dn_gdn_gates_bwd(a_.data_ptr(), b_.data_ptr(), A32.data_ptr(), d32.data_ptr(), dg.data_ptr(),
                                     dbeta.data_ptr(), B, Lq, Hv, _DT[a_.dtype], da.data_ptr(), db.data_ptr(), dA.data_ptr(),
                                     dD.data_ptr(), _stream()), "dn_gdn_gates_bwd")
        ta, tb, tA, tD = ctx.like
        return da.to(ta), db.to(tb), dA.to(tA), dD.to(tD)


def gdn_gates(a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor):
    """``g = -exp(A_log) * softplus(a + dt_bias)`` and ``beta = sigmoid(b)`` for (B, L, Hv) pre-activations and
    per-head parameters (Hv): the fp32 per-head scalar gates ``chunk_gdn`` takes."""
    if a.dim() != 3 or tuple(b.shape) != tuple(a.shape):
        raise ValueError(f"a and b must both be (B, L, Hv), got {tuple(a.shape)} and {tuple(b.shape)}.")
    if A_log.numel() != a.shape[2] or dt_bias.numel() != a.shape[2]:
        raise ValueError(f"A_log and dt_bias must have Hv = {a.shape[2]} elements.")
    _require_cuda(a, b, A_log, dt_bias)
    return _Gates.apply(a, b, A_log.reshape(-1), dt_bias.reshape(-1))


class _GatedNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, z, weight, eps):
        lib = L.lib()
        V = o.shape[-1]
        o_, z_ = o.contiguous(), z.to(o.dtype).contiguous()
        w32 = _f32(weight)
        rows = o_.numel() // V
        y = torch.empty_like(o_)
        L.check(lib.dn_gated_rmsnorm_fwd(o_.data_ptr(), z_.data_ptr(), w32.data_ptr(), rows, V, _DT[o_.dtype], float(eps),
                                         y.data_ptr(), _stream()), "dn_gated_rmsnorm_fwd")
        ctx.save_for_backward(o_, z_, w32)
        ctx.eps, ctx.like = float(eps), (z.dtype, weight.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = L.lib()
        o_, z_, w32 = ctx.saved_tensors
        V = o_.shape[-1]
        rows = o_.numel() // V
        dy = dy.to(o_.dtype).contiguous()
        d_o, d_z = torch.empty_like(o_), torch.empty_like(z_)
        dw = torch.empty_like(w32)
        n = lib.dn_gated_rmsnorm_scratch_bytes(rows, V)
        scratch = torch.empty(n, dtype=torch.uint8, device=o_.device)
        L.check(lib.dn_gated_rmsnorm_bwd(o_.data_ptr(), z_.data_ptr(), w32.data_ptr(), rows, V, _DT[o_.dtype], ctx.eps,
                                         dy.data_ptr(), d_o.data_ptr(), d_z.data_ptr(), dw.data_ptr(), scratch.data_ptr(), n,
                                         _stream()), "dn_gated_rmsnorm_bwd")
        tz, tw = ctx.like
        return d_o, d_z.to(tz), dw.to(tw), None


def gated_rmsnorm(o: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """``weight * rmsnorm(o) * silu(z)`` over the last dimension (a value head, 64 or 128 wide); ``o`` and ``z``
    have the same shape (..., V) and the result has ``o``'s shape and dtype.  The normalised value is rounded
    to ``o``'s dtype before the weight is applied, as the Qwen3.5 layer does."""
    if tuple(o.shape) != tuple(z.shape):
        raise ValueError(f"o and z must have the same shape, got {tuple(o.shape)} and {tuple(z.shape)}.")
    if o.shape[-1] not in (64, 128) or weight.numel() != o.shape[-1]:
        raise ValueError(f"the last dimension ({o.shape[-1]}) must be 64 or 128 and match weight ({weight.numel()}).")
    if o.dtype not in _DT:
        raise ValueError(f"o dtype {o.dtype} must be float32 or bfloat16.")
    _require_cuda(o, z, weight)
    return _GatedNorm.apply(o, z, weight.reshape(-1), eps)
