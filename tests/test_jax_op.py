"""The JAX front end (custom_vjp over XLA FFI custom calls).  Skipped where jax is not installed (it is not
in the image this package is developed on); where it is, and a GPU is present, the JAX operator is compared
with the CPU oracle like the torch front end."""
import os

import numpy as np
import pytest

jax = pytest.importorskip("jax", reason="jax is not installed: the optional JAX front end is not exercised")
pytestmark = pytest.mark.gpu


def test_jax_chunk_gdn2_matches_oracle():
    import torch
    from deltanet_b200 import jax_op
    from oracle import delta_oracle as O
    if not os.path.exists(jax_op._FFI_PATH):
        pytest.skip("the XLA FFI shim is not built (deltanet-tpu_b200/csrc/build_ffi.sh)")
    import jax.numpy as jnp
    B, L, Hk, Hv, K, V = 1, 384, 2, 4, 128, 128
    q, k, v, g, b, w = O.make_inputs(501, B, L, Hk, Hv, K, V, qkv_scale=0.5)
    seg = torch.tensor([0] * 200 + [1] * 184, dtype=torch.int32)
    leaves = [t.clone().requires_grad_() for t in (q, k, v, g, b, w)]
    o_ref = O.chunk_gdn2(*leaves, segment_ids=seg, chunk_size=128, precision="fp32", qk_l2norm=True)
    do = torch.randn(o_ref.shape, generator=torch.Generator().manual_seed(1))
    g_ref = torch.autograd.grad((o_ref * do).sum(), leaves)
    args = [jnp.asarray(t.numpy()) for t in (q, k, v, g, b, w)]
    f = lambda *a: jax_op.chunk_gdn2(*a, segment_ids=jnp.asarray(seg.numpy()), chunk_size=128, precision="fp32", qk_l2norm=True)
    o, vjp = jax.vjp(f, *args)
    grads = vjp(jnp.asarray(do.numpy()))
    assert O.rel_l2(np.asarray(o), o_ref.detach()) < 2e-4
    for a, r in zip(grads, g_ref):
        assert O.rel_l2(np.asarray(a), r) < 2e-4
