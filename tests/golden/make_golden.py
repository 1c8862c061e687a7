"""Generate the golden vectors in this folder by executing the reference's own code.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py /path/to/reference

It installs the numpy stand-in (``jax_numpy_standin.py``) for the array library the
reference imports, imports the reference package from ``<reference>/src`` unmodified,
and records inputs and outputs of:

* ``token_serial_gdn2``                      (reference.py:18)  -- the reference's ground truth,
* ``chunk_gdn2`` through its kernel bodies   (gdn2.py:1772; prepass/state kernels 115-769
  run by the stand-in's grid interpreter), forward AND the registered backward rule,
  in fp32 and bf16 precision, with the saved prepass residuals,
* ``chunk_gdn`` with per-value-head scalar gates (variants.py:17),
* ``chunk_gdn2(fuse_prologue=True)`` on an unaligned length,
* ``gdn2_decode_step`` with a bf16 state (gdn2.py:2289).

The tests never need the reference: they read the ``.npz`` files written here.
"""
from __future__ import annotations

import os
import sys
import warnings

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def sig(x):
    return (1.0 / (1.0 + np.exp(-x))).astype(np.float32)


def draw(rng, B, L, Hk, Hv, K, V, scale=0.1):
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    q, k, v = f(B, L, Hk, K) * scale, f(B, L, Hk, K) * scale, f(B, L, Hv, V) * scale
    b = sig(f(B, L, Hk, K) * 0.39)
    w = sig(f(B, L, Hv, V) * 0.39)
    g = -np.exp(f(B, L, Hk, K) * 0.39 - 1.0).astype(np.float32)
    return q, k, v, g, b, w


def fuse_state(s, Hk, G):
    B, Hv, K, V = s.shape
    return s.reshape(B, Hk, G, K, V).transpose(0, 1, 3, 2, 4).reshape(B, Hk, K, G * V)


def main(ref_root):
    warnings.simplefilter("ignore")
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.join(ref_root, "src"))
    import jax_numpy_standin as S
    S.install()
    import deltanet_tpu as D
    from deltanet_tpu.reference import token_serial_gdn2

    A = lambda x: None if x is None else np.asarray(x)
    save = lambda name, **kw: np.savez_compressed(os.path.join(HERE, name), **{k: v for k, v in kw.items() if v is not None})

    # ---- 1. the small fp32 forward case: token-serial ground truth, K=V=64
    rng = np.random.default_rng(1001)
    B, L, Hk, Hv, K, V = 1, 256, 2, 4, 64, 64
    q, k, v, g, b, w = draw(rng, B, L, Hk, Hv, K, V, scale=1.0)
    seg = np.array([0] * 128 + [1] * 128, dtype=np.int32)
    o, fs = token_serial_gdn2(q, k, v, g, b, w, segment_ids=seg, output_final_state=True, qk_l2norm=True)
    save("token_serial_small_fp32.npz", q=q, k=k, v=v, g=g, b=b, w=w, seg=seg, out=A(o), final_state=A(fs))

    # ---- 2/3. public chunked API through the kernel bodies, fwd + registered bwd
    rng = np.random.default_rng(1002)
    B, L, Hk, Hv, K, V = 1, 256, 1, 2, 128, 128
    G = Hv // Hk
    q, k, v, g, b, w = draw(rng, B, L, Hk, Hv, K, V)
    seg = np.array([0] * 90 + [1] * 166, dtype=np.int32)          # boundary inside chunk 0
    init = (rng.standard_normal((B, Hv, K, V)) * 0.1).astype(np.float32)
    do = rng.standard_normal((B, L, Hv, V)).astype(np.float32)
    dfs = (rng.standard_normal((B, Hv, K, V)) * 0.1).astype(np.float32)
    o_ts, fs_ts = token_serial_gdn2(q, k, v, g, b, w, segment_ids=seg, initial_state=init,
                                    output_final_state=True, scale=1.0)
    rec = dict(q=q, k=k, v=v, g=g, b=b, w=w, seg=seg, init=init, do=do, dfs=dfs,
               out_token_serial=A(o_ts), fs_token_serial=A(fs_ts))
    for prec in ("fp32", "bf16"):
        for rc in (False, True):
            S.TAPE.clear()
            o, fs = D.chunk_gdn2(q, k, v, g, b, w, segment_ids=seg, initial_state=init,
                                 output_final_state=True, precision=prec, scale=1.0,
                                 recompute_states=rc)
            op, args, res = S.TAPE[-1]
            grads = op.bwd(res, (do.reshape(B, L, Hk, G * V), fuse_state(dfs, Hk, G)))
            dq, dk, dv, dg, db, dw, _, dinit = grads
            tag = f"{prec}_stash"
            shapes = dict(dq=q, dk=k, dv=v, dg=g, db=b, dw=w)
            cur = {f"out_{tag}": A(o), f"fs_{tag}": A(fs)}
            for nm, x in zip(("dq", "dk", "dv", "dg", "db", "dw"), (dq, dk, dv, dg, db, dw)):
                cur[f"{nm}_{tag}"] = A(x).astype(np.float32).reshape(shapes[nm].shape)
            cur[f"dinit_{tag}"] = A(dinit).reshape(B, Hk, K, G, V).transpose(0, 1, 3, 2, 4).reshape(B, Hv, K, V)
            if rc:
                # the recompute mode is recorded as its largest relative deviation from the stashed mode
                dev = max(float(np.linalg.norm(cur[key] - rec[key]) / np.linalg.norm(rec[key])) for key in cur)
                rec[f"recompute_vs_stash_maxrel_{prec}"] = np.float64(dev)
                continue
            rec.update(cur)
            if not rc and prec == "fp32":
                # saved prepass residuals, exec-head layout (B,Hk,NC,C,.)
                names = ("W", "U", "M", "qe", "ke", "lambda_end")
                for nm, x in zip(names, res[7:13]):
                    rec[f"res_{nm}"] = A(x).astype(np.float32)
                rec["res_T"] = A(res[16]).astype(np.float32)
                rec["res_states"] = A(res[14]).astype(np.float32)
    save("chunk_api_k128.npz", **rec)

    # ---- 4. scalar per-value-head gates (the Gated DeltaNet layout), fp32, fwd + bwd
    rng = np.random.default_rng(1003)
    B, L, Hk, Hv, K, V = 2, 256, 1, 2, 128, 128
    q, k, v, _, _, _ = draw(rng, B, L, Hk, Hv, K, V)
    gs = -np.exp(rng.standard_normal((B, L, Hv)).astype(np.float32) * 0.39 - 1.0).astype(np.float32)
    beta = sig(rng.standard_normal((B, L, Hv)).astype(np.float32))
    seg = np.stack([np.repeat(np.arange(4, dtype=np.int32), [40, 100, 16, 100]),
                    np.repeat(np.arange(2, dtype=np.int32), [128, 128])])
    do = rng.standard_normal((B, L, Hv, V)).astype(np.float32)
    S.TAPE.clear()
    o, fs = D.chunk_gdn(q, k, v, gs, beta, segment_ids=seg, output_final_state=True,
                        precision="fp32", scale=1.0)
    op, args, res = S.TAPE[-1]
    grads = op.bwd(res, (do, np.zeros((B, Hv, K, V), np.float32)))
    dq, dk, dv, dg, db, dw, _, _ = grads
    o_ts = token_serial_gdn2(q, k, v, gs, beta, beta, segment_ids=seg, scale=1.0)
    save("gdn_scalar_gates_hv.npz", q=q, k=k, v=v, g=gs, beta=beta, seg=seg, do=do, out=A(o),
         final_state=A(fs), out_token_serial=A(o_ts), dq=A(dq), dk=A(dk), dv=A(dv),
         dg=A(dg).sum(-1), dbeta=A(db).sum(-1) + A(dw).sum(-1))

    # ---- 5. fused prologue on an unaligned length, fp32, fwd + bwd
    rng = np.random.default_rng(1004)
    B, L, Hk, Hv, K, V = 1, 200, 1, 1, 128, 128
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    q, k, v = f(B, L, Hk, K), f(B, L, Hk, K), f(B, L, Hv, V)
    g, b, w = f(B, L, Hk, K) * 0.5 - 1.0, f(B, L, Hk, K), f(B, L, Hv, V)
    do = f(B, L, Hv, V)
    S.TAPE.clear()
    o = D.chunk_gdn2(q, k, v, g, b, w, precision="fp32", qk_l2norm=True, fuse_prologue=True)
    op, args, res = S.TAPE[-1]
    do_pad = np.concatenate([do, np.zeros((B, 56, Hv, V), np.float32)], 1)
    grads = op.bwd(res, do_pad)
    o_ts = token_serial_gdn2(q, k, v, g, b, w, qk_l2norm=True, fuse_prologue=True)
    save("fused_prologue_unaligned.npz", q=q, k=k, v=v, g=g, b=b, w=w, do=do, out=A(o),
         out_token_serial=A(o_ts), **{nm: A(x)[:, :L] for nm, x in zip(("dq", "dk", "dv", "dg", "db", "dw"), grads[:6])})

    # ---- 6. decode step with a bf16 state
    import ml_dtypes
    rng = np.random.default_rng(1005)
    B, Hk, Hv, K, V = 2, 2, 4, 128, 128
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    q, k, v = f(B, Hk, K), f(B, Hk, K), f(B, Hv, V)
    b, w = sig(f(B, Hk, K) * 0.39), sig(f(B, Hv, V) * 0.39)
    g = -np.exp(f(B, Hk, K) * 0.39 - 1.0).astype(np.float32)
    state = (f(B, Hv, K, V) * 0.1).astype(ml_dtypes.bfloat16)
    reset = np.array([False, True])
    o, ns = D.gdn2_decode_step(q, k, v, g, b, w, state, reset=reset, qk_l2norm=True, state_dtype="bfloat16")
    o32, ns32 = D.gdn2_decode_step(q, k, v, g, b, w, state.astype(np.float32), qk_l2norm=True)
    save("decode_step_bf16_state.npz", q=q, k=k, v=v, g=g, b=b, w=w, state=state.astype(np.float32),
         reset=reset, out=A(o), new_state=A(ns).astype(np.float32), out_fp32=A(o32), new_state_fp32=A(ns32))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path of a checkout of the reference project>")
    main(sys.argv[1])
