"""Variant adapters: Gated DeltaNet, Kimi Delta Attention, GLA and DeltaNet on top of
``chunk_gdn2`` / ``gdn2_decode_step``.

Same names and keyword arguments as ``src/deltanet_tpu/variants.py`` of the reference
(chunk_gdn 17-88, chunk_kda 91-161, chunk_gla 164-221, chunk_delta_rule 224-285, decode
steps 308-417).  The chunk adapters additionally forward ``initial_state_segment_id`` so
that a packed sequence can be split across calls or GPUs through them as well.
"""
from __future__ import annotations

import torch

from .gdn2 import chunk_gdn2, gdn2_decode_step


def _check_scalar_beta(beta):
    if beta.dim() == 4 and beta.shape[-1] > 1:
        raise ValueError(
            f"beta must be a per-head scalar gate with shape (B, L, H) or (B, L, H, 1); "
            f"channel-wise beta with shape {tuple(beta.shape)} is not supported.")


def _const_gate(like, value, dims, dtype=torch.float32):
    """A gate that is one constant for all heads and channels: shape (B, L, 1) (or (B, 1) for decode).

    The reference writes ``zeros_like(k)`` / ``ones_like(v)`` here (variants.py:206-207, 271) and
    relies on its compiler to fold them; the kernels read a one-head scalar gate natively, so nothing
    of the size of k or v is materialised.
    """
    return torch.full(tuple(like.shape[:dims]) + (1,), float(value), dtype=dtype if dtype in (torch.float32, torch.bfloat16) else torch.float32, device=like.device)


def chunk_gdn(q, k, v, g, beta, *, segment_ids=None, cu_seqlens=None, initial_state=None,
              output_final_state=False, chunk_size=128, precision="bf16", scale=None,
              qk_l2norm=False, fallback_scan=False, is_inference=False, fuse_prologue=False,
              recompute_states=False, initial_state_segment_id=None):
    """Gated DeltaNet: scalar log-decay per head ``g`` and shared gate ``beta``."""
    _check_scalar_beta(beta)
    return chunk_gdn2(q, k, v, g, beta, beta, segment_ids=segment_ids, cu_seqlens=cu_seqlens,
                      initial_state=initial_state, output_final_state=output_final_state,
                      chunk_size=chunk_size, precision=precision, scale=scale, qk_l2norm=qk_l2norm,
                      fallback_scan=fallback_scan, is_inference=is_inference,
                      fuse_prologue=fuse_prologue, recompute_states=recompute_states,
                      initial_state_segment_id=initial_state_segment_id)


def chunk_kda(q, k, v, g, beta, *, segment_ids=None, cu_seqlens=None, initial_state=None,
              output_final_state=False, chunk_size=128, precision="bf16", scale=None,
              qk_l2norm=False, fallback_scan=False, is_inference=False, fuse_prologue=False,
              recompute_states=False, initial_state_segment_id=None):
    """Kimi Delta Attention: channel-wise log-decay ``g`` and shared gate ``beta``."""
    _check_scalar_beta(beta)
    return chunk_gdn2(q, k, v, g, beta, beta, segment_ids=segment_ids, cu_seqlens=cu_seqlens,
                      initial_state=initial_state, output_final_state=output_final_state,
                      chunk_size=chunk_size, precision=precision, scale=scale, qk_l2norm=qk_l2norm,
                      fallback_scan=fallback_scan, is_inference=is_inference,
                      fuse_prologue=fuse_prologue, recompute_states=recompute_states,
                      initial_state_segment_id=initial_state_segment_id)


def chunk_gla(q, k, v, g, *, segment_ids=None, cu_seqlens=None, initial_state=None,
              output_final_state=False, chunk_size=128, precision="bf16", scale=None,
              qk_l2norm=False, fallback_scan=False, is_inference=False, recompute_states=False):
    """Gated Linear Attention: GDN-2 with erase gate 0 and write gate 1."""
    b = _const_gate(k, 0.0, 2, g.dtype)
    w = _const_gate(v, 1.0, 2, g.dtype)
    return chunk_gdn2(q, k, v, g, b, w, segment_ids=segment_ids, cu_seqlens=cu_seqlens,
                      initial_state=initial_state, output_final_state=output_final_state,
                      chunk_size=chunk_size, precision=precision, scale=scale, qk_l2norm=qk_l2norm,
                      fallback_scan=fallback_scan, is_inference=is_inference,
                      recompute_states=recompute_states)


def chunk_delta_rule(q, k, v, beta, *, segment_ids=None, cu_seqlens=None, initial_state=None,
                     output_final_state=False, chunk_size=128, precision="bf16", scale=None,
                     qk_l2norm=False, fallback_scan=False, is_inference=False, recompute_states=False):
    """DeltaNet: no decay (g = 0) and b = w = beta."""
    _check_scalar_beta(beta)
    g = _const_gate(k, 0.0, 2, beta.dtype)
    return chunk_gdn2(q, k, v, g, beta, beta, segment_ids=segment_ids, cu_seqlens=cu_seqlens,
                      initial_state=initial_state, output_final_state=output_final_state,
                      chunk_size=chunk_size, precision=precision, scale=scale, qk_l2norm=qk_l2norm,
                      fallback_scan=fallback_scan, is_inference=is_inference,
                      recompute_states=recompute_states)


def _validate_decode_beta(beta):
    msg = ("beta must be a per-head scalar gate with shape (B, H), (B, H, 1) or (B, 1, H); "
           f"channel-wise beta with shape {tuple(beta.shape)} is not supported.")
    if beta.dim() == 3:
        if beta.shape[1] == 1:
            beta = beta[:, 0]
        elif beta.shape[-1] > 1:
            raise ValueError(msg)
    elif beta.dim() == 4:
        if beta.shape[-1] > 1:
            raise ValueError(msg)
        if beta.shape[1] == 1:
            beta = beta[:, 0]
    return beta


def gdn_decode_step(q, k, v, g, beta, state, *, reset=None, scale=None, qk_l2norm=False, state_dtype=None):
    """Single-token Gated DeltaNet step."""
    beta = _validate_decode_beta(beta)
    return gdn2_decode_step(q, k, v, g, beta, beta, state, reset=reset, scale=scale,
                            qk_l2norm=qk_l2norm, state_dtype=state_dtype)


def kda_decode_step(q, k, v, g, beta, state, *, reset=None, scale=None, qk_l2norm=False, state_dtype=None):
    """Single-token Kimi Delta Attention step."""
    beta = _validate_decode_beta(beta)
    return gdn2_decode_step(q, k, v, g, beta, beta, state, reset=reset, scale=scale,
                            qk_l2norm=qk_l2norm, state_dtype=state_dtype)


def gla_decode_step(q, k, v, g, state, *, reset=None, scale=None, qk_l2norm=False, state_dtype=None):
    """Single-token Gated Linear Attention step."""
    one_tok = k[:, 0] if k.dim() == 4 else k
    return gdn2_decode_step(q, k, v, g, _const_gate(one_tok, 0.0, 1, g.dtype), _const_gate(one_tok, 1.0, 1, g.dtype), state, reset=reset,
                            scale=scale, qk_l2norm=qk_l2norm, state_dtype=state_dtype)


def delta_rule_decode_step(q, k, v, beta, state, *, reset=None, scale=None, qk_l2norm=False, state_dtype=None):
    """Single-token DeltaNet step (no decay)."""
    beta = _validate_decode_beta(beta)
    return gdn2_decode_step(q, k, v, _const_gate(k[:, 0] if k.dim() == 4 else k, 0.0, 1, beta.dtype), beta, beta, state, reset=reset, scale=scale,
                            qk_l2norm=qk_l2norm, state_dtype=state_dtype)
