"""The CPU oracle against vectors recorded from the reference's own code (tests/golden)."""
import os

import numpy as np
import pytest
import torch

from oracle import delta_oracle as O

T = lambda x: torch.from_numpy(np.asarray(x))


def load(golden_dir, name):
    d = np.load(os.path.join(golden_dir, name))
    return {k: d[k] for k in d.files}


def test_token_serial_small_fp32(golden_dir):
    d = load(golden_dir, "token_serial_small_fp32.npz")
    args = [T(d[n]) for n in "qkvgbw"]
    o, fs = O.token_serial_gdn2(*args, segment_ids=T(d["seg"]), output_final_state=True, qk_l2norm=True)
    assert O.rel_l2(o, d["out"]) < 2e-6
    assert O.rel_l2(fs, d["final_state"]) < 2e-6
    # the chunked restatement at the small configuration (chunk 64, K=V=64) hits the same answer
    o2, fs2 = O.chunk_gdn2(*args, segment_ids=T(d["seg"]), output_final_state=True, qk_l2norm=True,
                           chunk_size=64, precision="fp32")
    assert O.rel_l2(o2, d["out"]) < 1e-5
    assert O.rel_l2(fs2, d["final_state"]) < 1e-5


@pytest.mark.parametrize("prec,tol", [("fp32", 2e-6), ("bf16", 2e-3)])
def test_chunk_api_forward_and_grads(golden_dir, prec, tol):
    d = load(golden_dir, "chunk_api_k128.npz")
    args = [T(d[n]).clone().requires_grad_() for n in "qkvgbw"]
    init = T(d["init"]).clone().requires_grad_()
    o, fs = O.chunk_gdn2(*args, segment_ids=T(d["seg"]), initial_state=init, output_final_state=True,
                         precision=prec, scale=1.0)
    assert O.rel_l2(o, d[f"out_{prec}_stash"]) < tol
    assert O.rel_l2(fs, d[f"fs_{prec}_stash"]) < tol
    loss = (o * T(d["do"])).sum() + (fs * T(d["dfs"])).sum()
    grads = torch.autograd.grad(loss, args + [init])
    gtol = 5e-5 if prec == "fp32" else 2e-2
    for nm, gr in zip(("dq", "dk", "dv", "dg", "db", "dw", "dinit"), grads):
        assert O.rel_l2(gr, d[f"{nm}_{prec}_stash"]) < gtol, nm
    assert d[f"recompute_vs_stash_maxrel_{prec}"] < 1e-6


def test_chunk_api_intermediates(golden_dir):
    d = load(golden_dir, "chunk_api_k128.npz")
    q, k, v, g, b, w = (T(d[n]) for n in "qkvgbw")
    B, L, Hk, K = q.shape
    Hv, V = v.shape[2], v.shape[3]
    seg = O.canonical_segments(T(d["seg"])[None].to(torch.int32))
    C = 128
    for c in range(L // C):
        sl = slice(c * C, (c + 1) * C)
        im = O.chunk_intermediates(q[0, sl, 0], k[0, sl, 0], g[0, sl, 0], b[0, sl, 0],
                                   v[0, sl].reshape(C, Hv * V), w[0, sl].reshape(C, Hv * V), seg[0, sl])
        for nm, key in (("W", "W"), ("U", "U"), ("M", "M"), ("qe", "qe"), ("ke", "ke"), ("T", "T")):
            assert O.rel_l2(im[key], d[f"res_{nm}"][0, 0, c]) < 5e-6, (nm, c)
        assert O.rel_l2(im["lambda_end"], d["res_lambda_end"][0, 0, c, 0]) < 1e-6


def test_gdn_scalar_gates_hv(golden_dir):
    d = load(golden_dir, "gdn_scalar_gates_hv.npz")
    q, k, v, g, beta = (T(d[n]).clone().requires_grad_() for n in ("q", "k", "v", "g", "beta"))
    o, fs = O.chunk_gdn(q, k, v, g, beta, segment_ids=T(d["seg"]), output_final_state=True,
                        precision="fp32", scale=1.0)
    assert O.rel_l2(o, d["out"]) < 2e-6
    assert O.rel_l2(fs, d["final_state"]) < 2e-6
    grads = torch.autograd.grad((o * T(d["do"])).sum(), [q, k, v, g, beta])
    for nm, gr in zip(("dq", "dk", "dv", "dg", "dbeta"), grads):
        assert O.rel_l2(gr, d[nm]) < 5e-5, nm


def test_fused_prologue_unaligned(golden_dir):
    d = load(golden_dir, "fused_prologue_unaligned.npz")
    args = [T(d[n]).clone().requires_grad_() for n in "qkvgbw"]
    o = O.chunk_gdn2(*args, precision="fp32", qk_l2norm=True, fuse_prologue=True)
    assert O.rel_l2(o, d["out"]) < 2e-6
    grads = torch.autograd.grad((o * T(d["do"])).sum(), args)
    for nm, gr in zip(("dq", "dk", "dv", "dg", "db", "dw"), grads):
        assert O.rel_l2(gr, d[nm]) < 5e-5, nm


def test_decode_step(golden_dir):
    d = load(golden_dir, "decode_step_bf16_state.npz")
    args = [T(d[n]) for n in "qkvgbw"]
    st = T(d["state"]).to(torch.bfloat16)
    o, ns = O.decode_step(*args, st, reset=T(d["reset"]), qk_l2norm=True, state_dtype=torch.bfloat16)
    assert O.rel_l2(o, d["out"]) < 2e-6
    assert O.rel_l2(ns.float(), d["new_state"]) < 1e-3          # one bf16 ulp flips allowed
    o2, ns2 = O.decode_step(*args, st.float(), qk_l2norm=True)
    assert ns2.dtype == torch.float32
    assert O.rel_l2(o2, d["out_fp32"]) < 2e-6
    assert O.rel_l2(ns2, d["new_state_fp32"]) < 2e-6
