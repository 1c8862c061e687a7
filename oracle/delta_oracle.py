"""CPU oracle for the delta-rule recurrence core.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch-on-CPU code, the arithmetic of the reference
package's delta-rule path so that the CUDA kernels can be checked against it.
Nothing in the shipped package imports it: it is used by ``tests/``, by the smoke
check and by the CPU-baseline leg of the benchmark, and by nothing else.

Which reference code each function follows (paths inside the reference project):

* ``token_serial_gdn2``      -- src/deltanet_tpu/reference.py:55-173 (prologue 62-80, head
  repeat 82-91, gate broadcast 93-107, per-token step 123-148, initial carry 150-155).
* ``invert_unit_triangular`` -- src/deltanet_tpu/gdn2.py:67-111 (16x16 diagonal doubling,
  degree-7 outer polynomial, one Newton-Schulz step).
* ``chunk_intermediates``    -- src/deltanet_tpu/gdn2.py:772-899 (one chunk, one head: the
  cumulative decay, the A and M matrices built from 32x32 sub-blocks, T, W, U, the masked
  q/k factors) which is also what the Pallas prepass body gdn2.py:115-240 computes.
* ``chunked_scan_gdn2``      -- src/deltanet_tpu/gdn2.py:932-1000 (the scan over chunks and
  the carry between them, flags as in gdn2.py:1291-1302).
* ``chunk_gdn2``             -- the wrapper semantics of src/deltanet_tpu/gdn2.py:1969-2127
  and 2259-2286: gate clamp, gate broadcast, segment canonicalisation, padding to a
  multiple of the chunk, q/k normalisation rounded to the input dtype, output slicing.
* ``decode_step``            -- src/deltanet_tpu/gdn2.py:2393-2489.

Pinning: ``tests/golden/`` holds vectors produced by executing the reference's own
source files (under a small numpy stand-in for the array library they import) and
the oracle is checked against them in ``tests/test_oracle_golden.py``; it is also
checked against two independent third-party recurrences (transformers' Qwen3.5
torch reference and flash-linear-attention's naive KDA) in ``tests/test_oracle_pin.py``.

Everything is differentiable with torch autograd, which is how gradient oracles
are obtained (the reference differentiates the same functions with jax.vjp).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

SUB = 32  # sub-block edge of the intra-chunk factorisation (gdn2.py:793)


# --------------------------------------------------------------------------- helpers
class _NonPositiveGate(torch.autograd.Function):
    """g -> min(g, 0) whose gradient is passed where g <= 0 (gdn2.py:50-64)."""

    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return torch.where(x <= 0, x, torch.zeros_like(x))

    @staticmethod
    def backward(ctx, gout):
        (x,) = ctx.saved_tensors
        return torch.where(x <= 0, gout, torch.zeros_like(gout))


def nonpositive_gate(x: torch.Tensor) -> torch.Tensor:
    return _NonPositiveGate.apply(x)


def _np_clamp(x: torch.Tensor) -> torch.Tensor:
    """Plain clamp of an exponent to <= 0 (gdn2.py:38-41); subgradient 1 at 0."""
    return torch.where(x <= 0, x, torch.zeros_like(x))


def _bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype)


def _mm(a, b, bf16_operands: bool):
    """Matmul with fp32(+) accumulation; operands rounded to bf16 when asked."""
    if bf16_operands:
        return _bf16_round(a) @ _bf16_round(b)
    return a @ b


def rel_l2(a, b) -> float:
    a = torch.as_tensor(a).double().flatten()
    b = torch.as_tensor(b).double().flatten()
    return float((a - b).norm() / (b.norm() + 1e-12))


def _expand_gate(x, B, L, H_from, H_to, width):
    """(B,L,h[,c]) gate -> (B,L,H_to,width); heads 1/Hk/Hv, channels 1/width."""
    if x.dim() == 3:
        x = x.unsqueeze(-1)
    h = x.shape[2]
    if h != H_to:
        if h == 1:
            x = x.expand(B, L, H_to, x.shape[-1])
        else:
            x = x.repeat_interleave(H_to // h, dim=2)
    if x.shape[-1] != width:
        x = x.expand(B, L, H_to, width)
    return x


def segment_ids_from_cu_seqlens(cu_seqlens, L: int) -> torch.Tensor:
    cu = [int(c) for c in cu_seqlens]
    ids = torch.zeros(L, dtype=torch.int32)
    for d in range(len(cu) - 1):
        ids[cu[d]:cu[d + 1]] = d
    return ids


# --------------------------------------------------------------------------- token serial
def token_serial_gdn2(q, k, v, g, b, w, *, segment_ids=None, cu_seqlens=None,
                      initial_state=None, output_final_state=False, scale=None,
                      qk_l2norm=False, fuse_prologue=False):
    """One token at a time; the ground truth every reference test compares against."""
    B, L, Hk, K = q.shape
    Hv, V = v.shape[2], v.shape[3]
    if scale is None:
        scale = 1.0 / math.sqrt(K)
    if fuse_prologue:
        q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * scale
        k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        g = -torch.exp(torch.clamp(g, max=5.0))
        b = torch.sigmoid(b)
        w = torch.sigmoid(w)
    elif qk_l2norm:
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * scale
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    else:
        q = q * scale
    G = Hv // Hk
    if G > 1:
        q = q.repeat_interleave(G, dim=2)
        k = k.repeat_interleave(G, dim=2)
    g = _expand_gate(g, B, L, None, Hv, K)
    b = _expand_gate(b, B, L, None, Hv, K)
    w = _expand_gate(w, B, L, None, Hv, V)
    if segment_ids is not None:
        seg = segment_ids if segment_ids.dim() == 2 else segment_ids[None].expand(B, L)
    elif cu_seqlens is not None:
        seg = segment_ids_from_cu_seqlens(cu_seqlens, L)[None].expand(B, L)
    else:
        seg = torch.zeros(B, L, dtype=torch.int32)
    dt = q.dtype
    if initial_state is not None:
        S = initial_state.to(dt)
        prev = seg[:, 0].clone()
    else:
        S = torch.zeros(B, Hv, K, V, dtype=dt)
        prev = torch.full((B,), -1, dtype=seg.dtype)
    outs = []
    gc = nonpositive_gate(g)
    for t in range(L):
        fresh = (seg[:, t] != prev).view(B, 1, 1, 1)
        S = torch.where(fresh, torch.zeros_like(S), S)
        S = torch.exp(gc[:, t]).unsqueeze(-1) * S
        beta = b[:, t] * k[:, t]
        erase = (beta.unsqueeze(-1) * S).sum(2)
        v_new = w[:, t] * v[:, t] - erase
        S = S + k[:, t].unsqueeze(-1) * v_new.unsqueeze(2)
        outs.append((S * q[:, t].unsqueeze(-1)).sum(2))
        prev = seg[:, t]
    out = torch.stack(outs, dim=1)
    return (out, S) if output_final_state else out


# --------------------------------------------------------------------------- inverse
def invert_unit_triangular(A: torch.Tensor) -> torch.Tensor:
    """(I + A)^-1 for strictly lower-triangular A, by the reference's scheme."""
    C = A.shape[-1]
    blk = 16 if C >= 16 else C
    if C > 8 * blk:
        raise ValueError(f"Chunk size C={C} exceeds maximum supported (C <= {8 * blk})")
    eye = torch.eye(C, dtype=A.dtype)
    idx = torch.arange(C)
    on_diag = (idx[:, None] // blk) == (idx[None, :] // blk)
    D = torch.where(on_diag, A, torch.zeros_like(A))
    R = A - D
    N = -D
    P = eye + N
    cur = N
    for _ in range(max(0, int(math.ceil(math.log2(blk))) - 1)):
        cur = cur @ cur
        P = P + P @ cur
    Mx = P @ R
    M2 = Mx @ Mx
    M4 = M2 @ M2
    T = ((eye - Mx) @ (eye + M2)) @ (eye + M4) @ P
    return T @ (2.0 * eye - (eye + A) @ T)


# --------------------------------------------------------------------------- one chunk
def chunk_intermediates(q, k, g, b, v, w, seg, *, bf16_operands=False,
                        mask_lambda_by_doc=False, exact_inverse=False):
    """All per-chunk quantities for one head.

    q,k,g,b: (C,K); v,w: (C,Vw); seg: (C,) ints.  Returns a dict with Lambda, A, M,
    T, W, U, qe, ke, lambda_end.  ``exact_inverse`` swaps the reference's polynomial
    inverse for a triangular solve (the reference's own test treats them as equal).
    """
    C, K = q.shape
    NS = C // SUB
    dt = q.dtype
    same = seg[:, None] == seg[None, :]
    ones = torch.ones(C, C, dtype=dt)
    tril = torch.tril(same.to(dt)) if mask_lambda_by_doc else torch.tril(ones)
    Lam = tril @ g
    beta = b * k
    ar = torch.arange(SUB)
    strict_sub = ar[:, None] > ar[None, :]
    lower_sub = ar[:, None] >= ar[None, :]
    A_rows, M_rows = [], []
    for a in range(NS):
        sa, ea = a * SUB, (a + 1) * SUB
        ref_row = Lam[sa:sa + 1]
        row_fac = torch.exp(_np_clamp(Lam[sa:ea] - ref_row))
        bb = beta[sa:ea] * row_fac
        qq = q[sa:ea] * row_fac
        pa, pm = [], []
        for c in range(a):
            sc, ec = c * SUB, (c + 1) * SUB
            kk = k[sc:ec] * torch.exp(_np_clamp(ref_row - Lam[sc:ec]))
            pa.append(bb @ kk.T)
            pm.append(qq @ kk.T)
        La = Lam[sa:ea]
        dec = torch.exp(_np_clamp(La[:, None, :] - La[None, :, :]))
        zero = torch.zeros(SUB, SUB, dtype=dt)
        pa.append(torch.where(strict_sub, ((beta[sa:ea][:, None, :] * dec) * k[sa:ea][None]).sum(-1), zero))
        pm.append(torch.where(lower_sub, ((q[sa:ea][:, None, :] * dec) * k[sa:ea][None]).sum(-1), zero))
        if ea < C:
            pa.append(torch.zeros(SUB, C - ea, dtype=dt))
            pm.append(torch.zeros(SUB, C - ea, dtype=dt))
        A_rows.append(torch.cat(pa, 1))
        M_rows.append(torch.cat(pm, 1))
    A_raw = torch.cat(A_rows, 0)
    M_raw = torch.cat(M_rows, 0)
    io = torch.arange(C)
    A = torch.where((io[:, None] > io[None, :]) & same, A_raw, torch.zeros_like(A_raw))
    M = torch.where((io[:, None] >= io[None, :]) & same, M_raw, torch.zeros_like(M_raw))
    first_doc = (seg == seg[0])[:, None]
    last_doc = (seg == seg[-1])[:, None]
    eL = torch.exp(_np_clamp(Lam))
    X = torch.where(first_doc, beta * eL, torch.zeros_like(beta))
    qe = torch.where(first_doc, q * eL, torch.zeros_like(q))
    lam_end = Lam[-1:]
    ke = torch.where(last_doc, k * torch.exp(_np_clamp(lam_end - Lam)), torch.zeros_like(k))
    if exact_inverse:
        T = torch.linalg.solve_triangular(torch.eye(C, dtype=dt) + A, torch.eye(C, dtype=dt), upper=False)
    else:
        T = invert_unit_triangular(A)
    W = _mm(T, X, bf16_operands)
    U = _mm(T, w * v, bf16_operands)
    return dict(Lambda=Lam, A=A, M=M, T=T, W=W, U=U, X=X, qe=qe, ke=ke, lambda_end=lam_end[0])


def chunk_step(S_prev, prev_seg, q, k, g, b, v, w, seg, *, bf16_operands=False,
               state_fp32_matmul=False, mask_lambda_by_doc=False, exact_inverse=False):
    """Advance one head by one chunk; returns (S_next, S_entry, out, intermediates)."""
    im = chunk_intermediates(q, k, g, b, v, w, seg, bf16_operands=bf16_operands,
                             mask_lambda_by_doc=mask_lambda_by_doc, exact_inverse=exact_inverse)
    new_doc = bool(seg[0] != prev_seg)
    one_doc = bool(seg[0] == seg[-1])
    S_in = torch.zeros_like(S_prev) if new_doc else S_prev
    st_bf16 = bf16_operands and not state_fp32_matmul
    V_new = im["U"] - _mm(im["W"], S_in, st_bf16)
    out = _mm(im["qe"], S_in, st_bf16) + _mm(im["M"], V_new, bf16_operands)
    carried = S_in * torch.exp(_np_clamp(im["lambda_end"]))[:, None] if one_doc else torch.zeros_like(S_in)
    S_next = carried + _mm(im["ke"].T, V_new, st_bf16)
    im["V_new"] = V_new
    return S_next, S_in, out, im


def chunked_scan_gdn2(q, k, v, g, b, w, seg, chunk_size, *, precision="fp32",
                      initial_state=None, state_fp32_matmul=False,
                      mask_lambda_by_doc=False, exact_inverse=False,
                      return_intermediates=False):
    """The reference's chunked algorithm on already-prepared inputs.

    q,k,g,b: (B,L,Hv,K) and v,w: (B,L,Hv,V) with L a multiple of chunk_size, seg (B,L)
    canonical ids.  Returns (out, entry_states (NC,B,Hv,K,V), final_state[, per-chunk dicts]).
    """
    B, L, Hv, K = q.shape
    V = v.shape[-1]
    NC = L // chunk_size
    bf = precision.lower() in ("bf16", "bfloat16")
    dt = q.dtype
    out = torch.zeros(B, L, Hv, V, dtype=dt)
    entry = [[[None] * Hv for _ in range(B)] for _ in range(NC)]
    inter = {}
    finals = []
    for bi in range(B):
        row = []
        for h in range(Hv):
            S = initial_state[bi, h].to(dt) if initial_state is not None else torch.zeros(K, V, dtype=dt)
            prev = 0 if initial_state is not None else -1
            for c in range(NC):
                sl = slice(c * chunk_size, (c + 1) * chunk_size)
                S, S_in, o, im = chunk_step(
                    S, prev, q[bi, sl, h], k[bi, sl, h], g[bi, sl, h], b[bi, sl, h],
                    v[bi, sl, h], w[bi, sl, h], seg[bi, sl], bf16_operands=bf,
                    state_fp32_matmul=state_fp32_matmul, mask_lambda_by_doc=mask_lambda_by_doc,
                    exact_inverse=exact_inverse)
                prev = int(seg[bi, sl][-1])
                out[bi, sl, h] = o
                entry[c][bi][h] = S_in
                if return_intermediates:
                    inter[(bi, h, c)] = im
            row.append(S)
        finals.append(torch.stack(row))
    states = torch.stack([torch.stack([torch.stack(entry[c][bi]) for bi in range(B)]) for c in range(NC)])
    res = (out, states, torch.stack(finals))
    return res + (inter,) if return_intermediates else res


# --------------------------------------------------------------------------- wrapper semantics
def canonical_segments(seg: torch.Tensor, first_is_new: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Ids that increase by one wherever the raw id changes (gdn2.py:2087-2094)."""
    B, L = seg.shape
    base = torch.zeros(B, 1, dtype=torch.int32) if first_is_new is None else first_is_new.view(B, 1).to(torch.int32)
    if L > 1:
        chg = (seg[:, 1:] != seg[:, :-1]).to(torch.int32).cumsum(1).to(torch.int32)
        return base + torch.cat([torch.zeros(B, 1, dtype=torch.int32), chg], 1)
    return base.clone()


def chunk_gdn2(q, k, v, g, b, w, *, segment_ids=None, cu_seqlens=None, initial_state=None,
               initial_state_segment_id=None, output_final_state=False, chunk_size=128,
               precision="bf16", scale=None, qk_l2norm=False, fuse_prologue=False,
               stability_guard=False, stability_tau=1000.0, is_inference=False,
               state_fp32_matmul=False, mask_lambda_by_doc=False, exact_inverse=False,
               compute_dtype=None):
    """chunk_gdn2 as the reference's jnp chunked path evaluates it.

    ``compute_dtype`` (default: float32) is the dtype the chunk arithmetic runs in;
    pass torch.float64 for a high-precision oracle.  Inputs keep their own dtype for
    the rounding points the reference has (q/k normalisation is rounded back to the
    input dtype, the output is cast to v's dtype).
    """
    B, L0, Hk, K = q.shape
    Hv, V = v.shape[2], v.shape[3]
    cdt = compute_dtype or torch.float32
    out_dtype = v.dtype
    if scale is None:
        scale = 1.0 / math.sqrt(K)
    if not fuse_prologue:
        g = nonpositive_gate(g)
        if stability_guard:
            b = torch.clamp(b, min=0.0)
            g = torch.clamp(g, max=-1e-6)
    # segments
    if segment_ids is not None:
        seg = segment_ids if segment_ids.dim() == 2 else segment_ids[None].expand(B, L0)
        seg = seg.to(torch.int32)
    elif cu_seqlens is not None:
        seg = segment_ids_from_cu_seqlens(cu_seqlens, L0)[None].expand(B, L0)
    else:
        seg = torch.zeros(B, L0, dtype=torch.int32)
    first_new = None
    if initial_state is not None and initial_state_segment_id is not None:
        isid = torch.as_tensor(initial_state_segment_id, dtype=torch.int32).expand(B)
        first_new = (seg[:, 0] != isid).to(torch.int32)
    seg = canonical_segments(seg, first_new)
    # q/k normalisation, rounded to the input dtype unless the prologue is fused
    if fuse_prologue:
        qf, kf = q.to(cdt), k.to(cdt)
        qn = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6) * scale
        kn = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
        gf = -torch.exp(torch.clamp(g.to(cdt), max=5.0))
        if stability_guard:
            gf = torch.clamp(gf, max=-1e-6)
        bfv = torch.sigmoid(b.to(cdt))
        wf = torch.sigmoid(w.to(cdt))
    else:
        ndt = torch.float64 if q.dtype == torch.float64 else torch.float32
        qf, kf = q.to(ndt), k.to(ndt)
        if qk_l2norm:
            qn = (qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6) * scale).to(q.dtype)
            kn = (kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)).to(k.dtype)
        else:
            qn = (qf * scale).to(q.dtype)
            kn = k
        qn, kn = qn.to(cdt), kn.to(cdt)
        gf, bfv, wf = g.to(cdt), b.to(cdt), w.to(cdt)
    G = Hv // Hk
    if G > 1:
        qn = qn.repeat_interleave(G, dim=2)
        kn = kn.repeat_interleave(G, dim=2)
    gf = _expand_gate(gf, B, L0, None, Hv, K)
    bfv = _expand_gate(bfv, B, L0, None, Hv, K)
    wf = _expand_gate(wf, B, L0, None, Hv, V)
    vf = v.to(cdt)
    pad = (-L0) % chunk_size
    if pad:
        def zpad(x):
            return torch.cat([x, torch.zeros(B, pad, *x.shape[2:], dtype=x.dtype)], 1)
        qn, kn, vf, gf, bfv, wf = map(zpad, (qn, kn, vf, gf, bfv, wf))
        seg = torch.cat([seg, seg[:, -1:].expand(B, pad)], 1)
    init = None
    if initial_state is not None:
        init = initial_state.to(cdt)
        if first_new is not None:
            init = torch.where(first_new.view(B, 1, 1, 1).bool(), torch.zeros_like(init), init)
    out, _, final = chunked_scan_gdn2(qn, kn, vf, gf, bfv, wf, seg, chunk_size, precision=precision,
                                      initial_state=init, state_fp32_matmul=state_fp32_matmul,
                                      mask_lambda_by_doc=mask_lambda_by_doc, exact_inverse=exact_inverse)
    out = out[:, :L0].to(out_dtype)
    if output_final_state:
        final = final.to(torch.float32) if cdt == torch.float32 else final
        if stability_guard and is_inference:
            nrm = torch.sqrt((final ** 2).sum((-2, -1), keepdim=True) + 1e-6)
            final = final * torch.clamp(stability_tau / nrm, max=1.0)
        return out, final
    return out


# --------------------------------------------------------------------------- decode
def decode_step(q, k, v, g, b, w, state, *, reset=None, scale=None, qk_l2norm=False,
                state_dtype=None, stability_guard=False, stability_tau=1000.0):
    """Single-token update on (B,Hk,K)/(B,Hv,V) vectors and a (B,Hv,K,V) state."""
    out_dtype = v.dtype
    squeeze = q.dim() == 4
    if squeeze:
        q, k, v = q[:, 0], k[:, 0], v[:, 0]
        g = g[:, 0] if g.dim() in (3, 4) and g.shape[1] == 1 else g
        b = b[:, 0] if b.dim() in (3, 4) and b.shape[1] == 1 else b
        w = w[:, 0] if w.dim() in (3, 4) and w.shape[1] == 1 else w
    B, Hk, K = q.shape
    Hv, V = v.shape[1], v.shape[2]
    tgt = torch.float32 if state_dtype is None else state_dtype
    q, k, v, b, w = (x.float() for x in (q, k, v, b, w))
    g = torch.clamp(g.float(), max=0.0)
    if stability_guard:
        b = torch.clamp(b, min=0.0)
        g = torch.clamp(g, max=-1e-6)
    S = state.float()
    if reset is not None:
        r = torch.as_tensor(reset)
        r = r.view(-1, 1, 1, 1) if r.dim() > 0 else r
        S = torch.where(r.bool(), torch.zeros_like(S), S)
    if scale is None:
        scale = 1.0 / math.sqrt(K)
    if qk_l2norm:
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * scale
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    else:
        q = q * scale

    def widen(x, width):
        if x.dim() == 2:
            x = x.unsqueeze(-1)
        h = x.shape[1]
        if h != Hv:
            x = x.expand(B, Hv, x.shape[-1]) if h == 1 else x.repeat_interleave(Hv // h, dim=1)
        return x.expand(B, Hv, width) if x.shape[-1] != width else x

    q, k, g, b = widen(q, K), widen(k, K), widen(g, K), widen(b, K)
    w = widen(w, V)
    Sd = S * torch.exp(g).unsqueeze(-1)
    erase = ((b * k).unsqueeze(-1) * Sd).sum(2)
    v_new = w * v - erase
    Sn = Sd + k.unsqueeze(-1) * v_new.unsqueeze(2)
    o = (Sn * q.unsqueeze(-1)).sum(2).to(out_dtype)
    if squeeze:
        o = o[:, None]
    if stability_guard:
        nrm = torch.sqrt((Sn ** 2).sum((-2, -1), keepdim=True) + 1e-6)
        Sn = Sn * torch.clamp(stability_tau / nrm, max=1.0)
    return o, Sn.to(tgt)


# --------------------------------------------------------------------------- variants
def chunk_gdn(q, k, v, g, beta, **kw):
    return chunk_gdn2(q, k, v, g, beta, beta, **kw)


def chunk_kda(q, k, v, g, beta, **kw):
    return chunk_gdn2(q, k, v, g, beta, beta, **kw)


# --------------------------------------------------------------------------- synthetic inputs
def make_inputs(seed, B, L, Hk, Hv, K, V, *, qkv_dtype=torch.float32, qkv_scale=1.0,
                gate_layout="channel"):
    """Seeded inputs with the distributions the reference tests and benchmarks use.

    q,k,v ~ qkv_scale*N(0,1); b,w = sigmoid(0.39 N); g = -exp(0.39 N - 1)
    (tests/test_parity.py:18-26 of the reference use qkv_scale=0.1).
    gate_layout: "channel" (g,b at (B,L,Hk,K), w at (B,L,Hv,V)), "scalar_hv" (g,b,w at (B,L,Hv)).
    """
    gen = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen)
    q = (rn(B, L, Hk, K) * qkv_scale).to(qkv_dtype)
    k = (rn(B, L, Hk, K) * qkv_scale).to(qkv_dtype)
    v = (rn(B, L, Hv, V) * qkv_scale).to(qkv_dtype)
    if gate_layout == "channel":
        b = torch.sigmoid(rn(B, L, Hk, K) * 0.39)
        w = torch.sigmoid(rn(B, L, Hv, V) * 0.39)
        g = -torch.exp(rn(B, L, Hk, K) * 0.39 - 1.0)
    elif gate_layout == "scalar_hv":
        b = torch.sigmoid(rn(B, L, Hv) * 0.39)
        w = torch.sigmoid(rn(B, L, Hv) * 0.39)
        g = -torch.exp(rn(B, L, Hv) * 0.39 - 1.0)
    else:
        raise ValueError(gate_layout)
    return q, k, v, g, b, w
