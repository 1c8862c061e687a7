"""The allocation-free forward prepass (dn_prepass_fwd_static).

Some callers of the library cannot allocate device memory at the point where they call it (a
runtime whose call handlers may not allocate, a serving loop with a frozen memory plan, a
sandboxed plugin), so they cannot supply the scratch buffer dn_prepass_fwd wants.  This entry point
works out of a fixed array inside the library instead.  The test calls it through the C ABI twice
in a row -- the array keeps the first call's contents, which must not leak into the second -- and
compares every output with the regular entry point's on the same inputs.  It is collected last so
that a run stopping at the first failure has already run everything else, and it passes both alone
in a fresh process and after the other tests.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(lib, L, shape, ins, seg, static):
    dev = ins[0].device
    block = torch.full((lib.dn_residual_bytes(shape),), 0x7F, dtype=torch.uint8, device=dev)
    res = L.Residuals()
    L.check(lib.dn_residual_carve(shape, block.data_ptr(), res), "dn_residual_carve")
    st = torch.cuda.current_stream().cuda_stream
    ptrs = [t.data_ptr() for t in ins] + [seg.data_ptr()]
    if static:
        L.check(lib.dn_prepass_fwd_static(shape, *ptrs, res, st), "dn_prepass_fwd_static")
    else:
        n = lib.dn_scratch_bytes(shape, 0, 0)
        scratch = torch.empty(n, dtype=torch.uint8, device=dev)
        L.check(lib.dn_prepass_fwd(shape, *ptrs, res, scratch.data_ptr(), n, st), "dn_prepass_fwd")
    torch.cuda.synchronize()
    return block


@pytest.mark.parametrize("prec,K,V,C", [("bf16", 128, 128, 128), ("fp32", 64, 64, 64)])
def test_static_scratch_prepass_matches_regular_entry_point(prec, K, V, C):
    from deltanet_b200 import _lib as L
    from oracle import delta_oracle as O
    lib = L.lib()
    B, Ln, Hk, Hv = 2, 320, 2, 4
    seg = torch.tensor([0] * 100 + [1] * 220, dtype=torch.int32)[None].expand(B, Ln).contiguous().cuda()
    shape = L.Shape(B=B, L=Ln, Hk=Hk, Hv=Hv, K=K, V=V, chunk=C, g_heads=Hk, g_cols=K, b_heads=Hk, b_cols=K,
                    w_heads=Hv, w_cols=V, qkv_dtype=L.DN_F32, gate_dtype=L.DN_F32,
                    precision=L.DN_PREC_BF16 if prec == "bf16" else L.DN_PREC_FP32,
                    flags=L.DN_QK_L2NORM, scale=K ** -0.5)
    assert lib.dn_static_scratch_bytes() == 32 << 20
    for seed in (31, 32):                                        # two calls in a row, different data
        ins = [t.cuda().contiguous() for t in O.make_inputs(seed, B, Ln, Hk, Hv, K, V)]
        ref = _run(lib, L, shape, ins, seg, static=False)
        got = _run(lib, L, shape, ins, seg, static=True)
        assert torch.equal(got, ref)                             # same kernels, same inputs: bit-identical


def test_static_scratch_rejects_shapes_beyond_the_array():
    from deltanet_b200 import _lib as L
    lib = L.lib()
    B, Ln, Hk, Hv, K, V = 4, 4096, 8, 16, 128, 128               # fp32 path at K=V=128: far more than 32 MiB
    shape = L.Shape(B=B, L=Ln, Hk=Hk, Hv=Hv, K=K, V=V, chunk=128, g_heads=Hk, g_cols=K, b_heads=Hk, b_cols=K,
                    w_heads=Hv, w_cols=V, qkv_dtype=L.DN_F32, gate_dtype=L.DN_F32, precision=L.DN_PREC_FP32,
                    flags=0, scale=K ** -0.5)
    one = torch.zeros(16, device="cuda")
    res = L.Residuals(*([one.data_ptr()] * 8))
    rc = lib.dn_prepass_fwd_static(shape, *([one.data_ptr()] * 7), res, None)
    assert rc == 7 and b"static" in lib.dn_status_string(rc)
