"""Sequence-parallel chunk_gdn2: one contiguous shard of a long packed sequence per rank.

The reference has no sequence-parallel implementation; it provides the hooks
(``initial_state`` / ``output_final_state`` / ``initial_state_segment_id``,
``src/deltanet_tpu/gdn2.py:2081-2085``).  Chaining those serially would make every rank wait for
the whole state pass of its predecessor.  Two facts make the chain cheap instead:

* the state pass of a shard is affine in the incoming state, ``S_out = P S_in + Q`` per (batch, exec
  head), and P comes out of the SAME launch as Q: K extra columns that start from the identity with
  U = 0 (the recurrence acts on every value column independently);
* whatever a shard computes after its first document boundary does not depend on the incoming state
  at all (and, going backwards, nothing before its last boundary depends on the incoming cotangent).

  forward   1. every rank: prepass, then ONE state pass from a zero state that writes outputs and
               chunk states for the whole shard (final after the first boundary, provisional
               before it) and yields Q and P;
            2. exchange: one all-gather of every shard's (P, Q) and edge ids; rank r composes the
               maps of shards 0..r-1 itself (zeroing the state where the next shard starts a new
               document) and gets its S_in; P S_in + Q is the shard's final state.  (Or, with
               exchange="p2p": rank r receives S_in from r-1 and sends P S_in + Q to r+1.);
            3. every rank: the state pass again from its true S_in, which stops at the first chunk
               that no longer depends on it.
  backward  the mirror image with the state cotangent: a reverse pass with zero incoming cotangent
            writes dV / dH for the whole shard and d_init0, the exchange (one all-gather, or hops
            from rank r to r-1) yields d_S_in = P^T d_final + d_init0, a second reverse pass from the true
            d_final stops where dH no longer depends on it, and the chunk-parallel backward runs
            over the shard.

With ``recompute_states`` nothing but the inputs, P and S_in survives the forward; the backward
rebuilds the prepass outputs and the chunk states first (what ``gdn2.py:1545-1630`` does per call).

The per-shard arithmetic is behind an ``ops`` object: ``CudaOps`` (the C-ABI kernels) on GPUs;
tests substitute CPU ops to exercise the exchange logic with the gloo backend.  Transfers use
``torch.distributed`` (NCCL over NVLink on a B200 box); what is received always lands in a local
buffer before any kernel reads it.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import _lib as L
from . import gdn2 as _g


# --------------------------------------------------------------------------------- chain helpers
class Chain:
    """Neighbour transfers along the sequence: rank r-1 <- r -> r+1."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self._pending = []          # (work, tensor) of sends in flight: kept alive until the call ends

    def _peer(self, r):
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def _send(self, y, r):
        y = y.contiguous()
        self._pending.append((dist.isend(y, dst=self._peer(r), group=self.group), y))

    def _recv(self, like, r):
        x = torch.empty_like(like)
        dist.irecv(x, src=self._peer(r), group=self.group).wait()      # stream-ordered for NCCL, blocking for gloo
        return x

    def drain(self):
        """Waits for this rank's sends (their buffers may be released afterwards)."""
        for work, _ in self._pending:
            work.wait()
        self._pending.clear()

    def forward(self, first_value, step):
        """first_value on rank 0, else what rank-1 sent; returns (received, produced); sends produced on."""
        x = first_value if self.rank == 0 else self._recv(first_value, self.rank - 1)
        y, y_next = step(x)
        if self.rank < self.size - 1:
            self._send(y_next, self.rank + 1)
        return x, y

    def backward(self, last_value, step):
        """Cotangents flow r+1 -> r.  last_value is this rank's own d_final_state (zeros if none): it is
        added to what rank+1 sends, so a loss on an intermediate rank's final_state is honoured too."""
        x = last_value
        if self.rank < self.size - 1:
            x = self._recv(last_value, self.rank + 1) + last_value
        y = step(x)
        if self.rank > 0:
            self._send(y, self.rank - 1)
        return x, y

    def gather_edges(self, edges):
        """all ranks' (B,2) [first raw id, last raw id] -> list indexed by rank (control metadata)."""
        out = [torch.empty_like(edges) for _ in range(self.size)]
        dist.all_gather(out, edges, group=self.group)
        return out

    def all_gather(self, tensors):
        """Every rank's list of tensors (4-byte elements, same shapes on all ranks) in ONE collective:
        returns a list indexed by rank of lists of tensors (views of one receive buffer)."""
        flat = torch.cat([t.contiguous().reshape(-1).view(torch.float32) for t in tensors])
        n = flat.numel()
        buf = torch.empty(self.size * n, dtype=torch.float32, device=flat.device)
        dist.all_gather_into_tensor(buf, flat, group=self.group)
        sizes = [t.numel() for t in tensors]
        return [[part.view(t.dtype).view(t.shape) for part, t in zip(torch.split(buf[r * n:(r + 1) * n], sizes), tensors)]
                for r in range(self.size)]


class LocalChain:
    """The same neighbour transfers between threads of ONE process (tests on a single device).

    Build the set with ``LocalChain.make(n)`` and run each rank's call in its own host thread; only
    host threads wait on each other, kernels never do.
    """

    def __init__(self, rank, size, shared):
        self.rank, self.size, self._s = rank, size, shared
        self._calls = 0

    @staticmethod
    def make(n):
        import queue
        import threading
        shared = dict(fwd=[queue.Queue() for _ in range(n)], bwd=[queue.Queue() for _ in range(n)],
                      edges=[None] * n, barrier=threading.Barrier(n))
        return [LocalChain(r, n, shared) for r in range(n)]

    @staticmethod
    def _handoff(y):
        return y.clone()            # (all threads of the process enqueue on the same stream: host order is device order)

    def forward(self, first_value, step):
        x = first_value if self.rank == 0 else self._s["fwd"][self.rank].get(timeout=120)
        y, y_next = step(x)
        if self.rank < self.size - 1:
            self._s["fwd"][self.rank + 1].put(self._handoff(y_next))
        return x, y

    def backward(self, last_value, step):
        x = last_value
        if self.rank < self.size - 1:
            x = self._s["bwd"][self.rank].get(timeout=120) + last_value
        y = step(x)
        if self.rank > 0:
            self._s["bwd"][self.rank - 1].put(self._handoff(y))
        return x, y

    def drain(self):
        pass

    def gather_edges(self, edges):
        self._s["edges"][self.rank] = edges
        self._s["barrier"].wait(timeout=120)
        return list(self._s["edges"])

    def all_gather(self, tensors):
        key = ("all_gather", self._calls)
        self._calls += 1
        slot = self._s.setdefault(key, [None] * self.size)
        slot[self.rank] = [self._handoff(t) for t in tensors]
        self._s["barrier"].wait(timeout=120)
        return [list(x) for x in slot]


def continues_from_previous(edges_prev, edges_mine):
    """(B,) bool: this shard's first token belongs to the same document as the previous shard's last."""
    return edges_prev[:, 1] == edges_mine[:, 0]


# --------------------------------------------------------------------------------- CUDA shard ops
class CudaOps:
    """Per-shard work through the C-ABI entry points (no torch arithmetic on the path)."""

    def __init__(self, *, chunk_size=128, precision="bf16", scale=None, qk_l2norm=False, fuse_prologue=False,
                 recompute_states=False):
        self.chunk, self.precision, self.scale = chunk_size, precision, scale
        self.l2, self.fuse, self.recompute = qk_l2norm, fuse_prologue, recompute_states

    # -- forward
    def prepare(self, q, k, v, g, b, w, seg_raw):
        lib = L.lib()
        B, Lq, Hk, K = q.shape
        Hv, V = v.shape[2], v.shape[3]
        qkv_dt, gate_dt = _g._common_dtype((q, k, v)), _g._common_dtype((g, b, w))
        q, k, v = (t.to(qkv_dt).contiguous() for t in (q, k, v))
        g, b, w = (t.to(gate_dt).contiguous() for t in (g, b, w))
        gh, gc = _g._gate_layout(g, K)
        bh, bc = _g._gate_layout(b, K)
        wh, wc = _g._gate_layout(w, V)
        flags = (L.DN_QK_L2NORM if self.l2 else 0) | (L.DN_FUSE_PROLOGUE if self.fuse else 0) | L.DN_HAS_INIT
        scale = self.scale if self.scale is not None else K ** -0.5
        shape = L.Shape(B=B, L=Lq, Hk=Hk, Hv=Hv, K=K, V=V, chunk=self.chunk, g_heads=gh, g_cols=gc, b_heads=bh,
                        b_cols=bc, w_heads=wh, w_cols=wc, qkv_dtype=_g._DT[qkv_dt], gate_dtype=_g._DT[gate_dt],
                        precision=_g._precision_code(self.precision), flags=flags, scale=float(scale))
        ex = L.Exec()
        L.check(lib.dn_exec_view(shape, ex), "dn_exec_view")
        seg = torch.empty(B, Lq, dtype=torch.int32, device=q.device)
        raw = seg_raw.to(device=q.device, dtype=torch.int32).contiguous()
        L.check(lib.dn_canonical_segments(raw.data_ptr(), None, seg.data_ptr(), B, Lq, _g._stream()), "segments")
        c = dict(shape=shape, ex=ex, seg=seg, ins=(q, k, v, g, b, w), dims=(B, Lq, Hk, Hv, K, V))
        self._prepass(c)
        return c

    def _prepass(self, c):
        """Runs the forward prepass into a fresh residual block (with T and room for the chunk states)."""
        lib, shape = L.lib(), c["shape"]
        q, k, v, g, b, w = c["ins"]
        block = torch.empty(lib.dn_residual_bytes(shape), dtype=torch.uint8, device=q.device)
        res = L.Residuals()
        L.check(lib.dn_residual_carve(shape, block.data_ptr(), res), "carve")
        n = max(lib.dn_scratch_bytes(shape, 0, 0), lib.dn_scratch_bytes(shape, 1, 0))
        scratch = torch.empty(n, dtype=torch.uint8, device=q.device)
        L.check(lib.dn_prepass_fwd(shape, q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), b.data_ptr(),
                                   w.data_ptr(), c["seg"].data_ptr(), res, scratch.data_ptr(), n, _g._stream()),
                "dn_prepass_fwd")
        c.update(res=res, block=block, scratch=scratch)

    def summary(self, c, skip_provisional=False):
        """``skip_provisional``: a correction pass (``finish`` without ``exact``) will follow, so the outputs of
        the chunks that depend on the incoming state need not be computed here."""
        B, Lq, Hk, Hv, K, V = c["dims"]
        q, v = c["ins"][0], c["ins"][2]
        c["out"] = torch.empty(B, Lq, Hv, V, dtype=v.dtype, device=q.device)
        Q = torch.empty(B, Hv, K, V, device=q.device)
        P = torch.empty(B, c["ex"].H, K, K, device=q.device)
        shape = c["shape"]
        if skip_provisional:
            shape = L.Shape.from_buffer_copy(shape)
            shape.flags |= L.DN_SP_SKIP_PROVISIONAL
        L.check(L.lib().dn_sp_summary(shape, c["res"], c["seg"].data_ptr(), c["out"].data_ptr(), Q.data_ptr(),
                                      P.data_ptr(), _g._stream()), "dn_sp_summary")
        return P, Q

    def apply(self, c, P, S_in, Q, transpose=False, keep=None):
        """op(P) S_in + Q; ``keep`` (B,) bool: batch rows where it is False come out as zeros."""
        B, Lq, Hk, Hv, K, V = c["dims"]
        H = c["ex"].H
        S_in = S_in.contiguous()
        out = torch.empty_like(S_in)
        if keep is not None:
            keep = keep.to(torch.uint8).contiguous()
        L.check(L.lib().dn_sp_apply(P.data_ptr(), S_in.data_ptr(), None if Q is None else Q.data_ptr(),
                                    out.data_ptr(), None if keep is None else keep.data_ptr(), B, H, Hv // H, K, V,
                                    1 if transpose else 0, _g._stream()), "dn_sp_apply")
        return out

    def finish(self, c, S_in, exact=False):
        """``exact``: the summary pass already started from the true incoming state (the first shard without
        an initial state), so there is nothing to correct."""
        c["S_in"] = S_in.contiguous()
        if not exact:
            L.check(L.lib().dn_sp_correct_fwd(c["shape"], c["res"], c["seg"].data_ptr(), c["S_in"].data_ptr(),
                                              c["out"].data_ptr(), _g._stream()), "dn_sp_correct_fwd")
        out = c.pop("out")
        if self.recompute:                                  # keep only what the backward cannot rebuild
            for name in ("res", "block", "scratch"):
                c.pop(name)
        return out

    # -- backward
    def bwd_summary(self, c, d_out):
        lib = L.lib()
        B, Lq, Hk, Hv, K, V = c["dims"]
        if "res" not in c:                                  # recompute_states: prepass outputs and chunk states again
            self._prepass(c)
            L.check(lib.dn_recompute_states(c["shape"], c["res"], c["seg"].data_ptr(), c["S_in"].data_ptr(),
                                            _g._stream()), "dn_recompute_states")
        ex, dev = c["ex"], d_out.device
        items = B * ex.H * ex.NC
        c["d_out"] = d_out.to(c["ins"][2].dtype).contiguous()
        c["dV"] = torch.empty(items * ex.chunk * ex.Vw, device=dev)
        c["dH"] = torch.empty(items * K * ex.Vw, device=dev)
        d_init0 = torch.empty(B, Hv, K, V, device=dev)
        L.check(lib.dn_state_bwd(c["shape"], c["res"], c["seg"].data_ptr(), c["d_out"].data_ptr(), None,
                                 c["dV"].data_ptr(), c["dH"].data_ptr(), d_init0.data_ptr(), _g._stream()), "dn_state_bwd")
        return d_init0

    def bwd_finish(self, c, d_final, exact=False):
        """``exact``: the incoming cotangent is zero (the last shard without a loss on its final state), which
        is what the zero-cotangent pass assumed."""
        lib = L.lib()
        q, k, v, g, b, w = c["ins"]
        d_final = d_final.contiguous()
        if not exact:
            L.check(lib.dn_sp_correct_bwd(c["shape"], c["res"], c["seg"].data_ptr(), c["d_out"].data_ptr(),
                                          d_final.data_ptr(), c["dV"].data_ptr(), c["dH"].data_ptr(), _g._stream()),
                    "dn_sp_correct_bwd")
        grads = [torch.empty_like(t) for t in (q, k, v, g, b, w)]
        sc = c["scratch"]
        L.check(lib.dn_prepass_bwd(c["shape"], q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), b.data_ptr(),
                                   w.data_ptr(), c["seg"].data_ptr(), c["res"], c["d_out"].data_ptr(), c["dV"].data_ptr(),
                                   c["dH"].data_ptr(), *[t.data_ptr() for t in grads], sc.data_ptr(), sc.numel(),
                                   _g._stream()), "dn_prepass_bwd")
        return grads


# --------------------------------------------------------------------------------- the sharded op
def shard_edges(seg_raw):
    return torch.stack([seg_raw[:, 0], seg_raw[:, -1]], dim=1).to(torch.int32).contiguous()


def sp_forward(ops, chain, tensors, seg_raw, initial_state, exchange="gather"):
    """Runs the three forward steps on this rank.  Returns (out, final_state, saved context)."""
    q, k, v, g, b, w = tensors
    B, Hv, K, V = q.shape[0], v.shape[2], q.shape[3], v.shape[3]
    c = ops.prepare(q, k, v, g, b, w, seg_raw)
    # (only the first shard without an initial state keeps what the summary pass writes before its first boundary)
    P, Q = ops.summary(c, skip_provisional=not (chain.rank == 0 and initial_state is None))
    if exchange == "gather":
        return _forward_gathered(ops, chain, c, P, Q, seg_raw, initial_state)
    edges = chain.gather_edges(shard_edges(seg_raw).to(q.device))
    r = chain.rank
    cont_in = continues_from_previous(edges[r - 1], edges[r]) if r > 0 else None
    cont_out = continues_from_previous(edges[r], edges[r + 1]) if r < chain.size - 1 else None
    first = initial_state if initial_state is not None else torch.zeros(B, Hv, K, V, device=q.device)

    def step(S_in):
        S_out = ops.apply(c, P, S_in, Q)                  # the state after this shard
        if cont_out is None:
            return S_out, None
        # what the next shard may keep of it: nothing where it starts a new document
        return S_out, S_out * cont_out.view(B, 1, 1, 1).to(S_out.dtype)

    S_in, final = chain.forward(first.float().contiguous(), step)
    # The send must have left before a kernel that fills every SM is enqueued behind it: the transfer's own
    # kernel needs room on an SM to start, and a persistent one-CTA-per-SM kernel (the chunk-parallel passes)
    # would hold it back until it ends - and the next rank with it.  The stream waits here, not the host.
    chain.drain()
    out = ops.finish(c, S_in, exact=(r == 0 and initial_state is None))
    c.update(P=P, cont_in=cont_in, exchange="p2p")
    return out, final, c


def _forward_gathered(ops, chain, c, P, Q, seg_raw, initial_state):
    """Step 2 of the forward as ONE collective: every rank learns every shard's affine map (P, Q) and edge ids and
    composes its predecessors' maps itself (r small launches on rank r) instead of waiting for r hops.  The
    first rank publishes its own final state P S_0 + Q in place of Q, so the others start from zero and the
    initial state does not travel.  It is the arithmetic of the hop-by-hop chain in the same order."""
    r, n = chain.rank, chain.size
    dev = P.device
    B = P.shape[0]
    S_in = None
    if r == 0:
        S_in = (initial_state if initial_state is not None else torch.zeros_like(Q)).float().contiguous()
        Q_pub = ops.apply(c, P, S_in, Q) if initial_state is not None else Q      # = this shard's final state
    else:
        Q_pub = Q
    got = chain.all_gather([P.contiguous(), Q_pub.contiguous(), shard_edges(seg_raw).to(dev)])
    edges = [x[2] for x in got]
    conts = [None] + [continues_from_previous(edges[j - 1], edges[j]) for j in range(1, n)]    # conts[j]: shard j continues j-1's document
    if r == 0:
        final = Q_pub
    else:
        S = got[0][1] * conts[1].view(B, 1, 1, 1).to(Q.dtype)                      # after shard 0; nothing of it where shard 1 starts a document
        for j in range(1, r):
            S = ops.apply(c, got[j][0], S, got[j][1], keep=conts[j + 1])           # the state after shard j, masked the same way for shard j+1
        S_in = S
        final = ops.apply(c, P, S_in, Q)
    out = ops.finish(c, S_in, exact=(r == 0 and initial_state is None))
    c.update(P=P, cont_in=conts[r], exchange="gather", P_all=[x[0] for x in got], conts=conts)
    return out, final, c


def _backward_gathered(ops, chain, c, d_out, d_final_state):
    """The mirror image: rank j publishes e_j = P_j^T (its own final-state cotangent) + d_init0_j; the cotangent of
    shard j's incoming state is then d_in_j = cont_j * (P_j^T d_in_{j+1} + e_j), which rank r evaluates for its
    successors j = n-1 .. r+1 itself."""
    r, n = chain.rank, chain.size
    B = d_out.shape[0]
    d_init0 = ops.bwd_summary(c, d_out)
    e_mine = d_init0 if d_final_state is None else ops.apply(c, c["P"], d_final_state.float().contiguous(), d_init0, transpose=True)
    got = chain.all_gather([e_mine.contiguous()])
    d_next = None                                                                  # d_in of the successor (None: zero)
    for j in range(n - 1, r, -1):
        if d_next is None:
            d_next = got[j][0] * c["conts"][j].view(B, 1, 1, 1).to(got[j][0].dtype)
        else:
            d_next = ops.apply(c, c["P_all"][j], d_next, got[j][0], transpose=True, keep=c["conts"][j])
    own = d_final_state.float() if d_final_state is not None else None
    x = d_next if own is None else (own if d_next is None else d_next + own)       # cotangent of this shard's final state
    if x is None:                                                                  # the last shard, no loss on its final state
        x = torch.zeros_like(d_init0)
        d_in = d_init0
        if c["cont_in"] is not None:
            d_in = d_in * c["cont_in"].view(B, 1, 1, 1).to(d_in.dtype)
    else:
        d_in = ops.apply(c, c["P"], x.contiguous(), d_init0, transpose=True, keep=c["cont_in"])
    grads = ops.bwd_finish(c, x, exact=(r == n - 1 and d_final_state is None))
    return grads, d_in


def sp_backward(ops, chain, c, d_out, d_final_state):
    """Mirror of sp_forward for the cotangents; returns (grads of q,k,v,g,b,w, d_initial_state)."""
    if c.get("exchange") == "gather":
        return _backward_gathered(ops, chain, c, d_out, d_final_state)
    B = d_out.shape[0]
    d_init0 = ops.bwd_summary(c, d_out)
    last = d_final_state if d_final_state is not None else torch.zeros_like(d_init0)

    def step(d_final):
        d_in = ops.apply(c, c["P"], d_final, d_init0, transpose=True)      # P^T d_final + d_init0
        if c["cont_in"] is not None:                                        # the previous shard's state was dropped
            d_in = d_in * c["cont_in"].view(B, 1, 1, 1).to(d_in.dtype)      # where this shard starts a document
        return d_in

    d_final, d_in = chain.backward(last.float().contiguous(), step)
    chain.drain()                                                           # (as in sp_forward)
    grads = ops.bwd_finish(c, d_final, exact=(chain.rank == chain.size - 1 and d_final_state is None))
    return grads, d_in


class _SPFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ops, chain, exchange, seg_raw, q, k, v, g, b, w, initial_state):
        out, final, c = sp_forward(ops, chain, (q, k, v, g, b, w), seg_raw, initial_state, exchange)
        chain.drain()
        ctx.ops, ctx.chain, ctx.c = ops, chain, c
        ctx.has_init = initial_state is not None
        ctx.set_materialize_grads(False)
        return out, final

    @staticmethod
    def backward(ctx, d_out, d_final):
        c = ctx.c
        if d_out is None:
            B, Lq, Hk, Hv, K, V = c["dims"]
            d_out = torch.zeros(B, Lq, Hv, V, device=c["seg"].device)
        (dq, dk, dv, dg, db, dw), d_in = sp_backward(ctx.ops, ctx.chain, c, d_out, d_final)
        ctx.chain.drain()
        return None, None, None, None, dq, dk, dv, dg, db, dw, (d_in if ctx.has_init else None)


def chunk_gdn2_sp(q, k, v, g, b, w, *, segment_ids: torch.Tensor, initial_state: Optional[torch.Tensor] = None,
                  group=None, chunk_size: int = 128, precision: str = "bf16", scale: Optional[float] = None,
                  qk_l2norm: bool = False, fuse_prologue: bool = False, recompute_states: bool = False,
                  exchange: str = "gather", ops=None, chain=None):
    """chunk_gdn2 on this rank's contiguous shard of a packed sequence split over the ranks of ``group``.

    ``segment_ids`` (B, L_shard) are the GLOBAL document ids of the shard's tokens (any change of id is
    a boundary, also across shards).  ``initial_state`` is used on the first rank only.  Returns
    ``(out, final_state)``; ``final_state`` is the state after this shard (the sequence's final state on
    the last rank) and is differentiable on every rank.  ``recompute_states`` keeps no prepass output or
    chunk state between forward and backward (``gdn2.py:1384-1386``).  Differentiable: backward runs the
    reverse chain, so every rank must take part.  ``exchange``: "gather" (one all-gather of the shards' affine
    maps per direction, each rank composes its predecessors' maps itself) or "p2p" (the state handed from rank
    to rank by send / recv, r hops before rank r can go on).
    """
    if exchange not in ("gather", "p2p"):
        raise ValueError(f"exchange must be 'gather' or 'p2p', got {exchange!r}")
    ops = ops or CudaOps(chunk_size=chunk_size, precision=precision, scale=scale, qk_l2norm=qk_l2norm,
                         fuse_prologue=fuse_prologue, recompute_states=recompute_states)
    chain = chain or Chain(group)
    return _SPFunction.apply(ops, chain, exchange, segment_ids, q, k, v, g, b, w, initial_state)
