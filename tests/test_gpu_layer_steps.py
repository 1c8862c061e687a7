"""The steps either side of the recurrence in a Gated DeltaNet layer (short convolution + SiLU + split,
gate activations, gated RMSNorm) against plain torch on the CPU, forward and every gradient, and the
whole layer core against transformers' Qwen3.5 torch reference, which is what the reference's own
layer example compares with (examples/qwen3_5_layer_parity.py:135-168 of the reference)."""
import pytest
import torch
import torch.nn.functional as F

from oracle import delta_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dn():
    import deltanet_b200
    return deltanet_b200


def conv_ref(mixed, w, bias, seg):
    """Depthwise causal conv + SiLU per document, in fp32: F.conv1d on each document's slice, left-padded with zeros."""
    B, L, D = mixed.shape
    W = w.shape[-1]
    out = torch.zeros(B, L, D, dtype=torch.float32)
    for b in range(B):
        bounds = [0] + [t for t in range(1, L) if seg is not None and seg[b, t] != seg[b, t - 1]] + [L]
        for s, e in zip(bounds[:-1], bounds[1:]):
            x = F.pad(mixed[b, s:e].float().t()[None], (W - 1, 0))
            y = F.conv1d(x, w.float().reshape(D, 1, W), None if bias is None else bias.float(), groups=D)
            out[b, s:e] = F.silu(y)[0].t()
    return out


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("W,with_bias,with_seg", [(4, False, False), (4, True, True), (3, False, True), (2, True, False)])
def test_qkv_producer(dn, dtype, tol, W, with_bias, with_seg):
    B, L, Hk, Hv, K, V = 2, 301, 2, 4, 128, 64
    D = 2 * Hk * K + Hv * V
    gen = torch.Generator().manual_seed(10 + W)
    mixed = torch.randn(B, L, D, generator=gen).to(dtype)
    w = torch.randn(D, 1, W, generator=gen) * 0.5
    bias = torch.randn(D, generator=gen) * 0.1 if with_bias else None
    seg = None
    if with_seg:
        seg = torch.zeros(B, L, dtype=torch.int32)
        seg[0, 1:] = 1            # a one-token document
        seg[0, 130:] = 7          # ids need not be consecutive
        seg[0, 132:] = 3          # a two-token document right before a run boundary
        seg[1, 128:] = 2          # boundary exactly at the start of a backward run
    leaves = [mixed.clone().requires_grad_(), w.clone().requires_grad_()] + ([bias.clone().requires_grad_()] if with_bias else [])
    ref = conv_ref(leaves[0], leaves[1], leaves[2] if with_bias else None, seg)
    gens = torch.Generator().manual_seed(99)
    dy = torch.randn(B, L, D, generator=gens).to(dtype).float()
    g_ref = torch.autograd.grad((ref * dy).sum(), leaves)
    dev = [mixed.cuda().requires_grad_(), w.cuda().requires_grad_()] + ([bias.cuda().requires_grad_()] if with_bias else [])
    q, k, v = dn.gdn_qkv_producer(dev[0], dev[1], dev[2] if with_bias else None, num_k_heads=Hk, num_v_heads=Hv,
                                  head_k_dim=K, head_v_dim=V, segment_ids=None if seg is None else seg.cuda())
    assert q.shape == (B, L, Hk, K) and v.shape == (B, L, Hv, V) and q.dtype == dtype
    got = torch.cat([q.reshape(B, L, -1), k.reshape(B, L, -1), v.reshape(B, L, -1)], -1)
    assert O.rel_l2(got.float().cpu(), ref.detach()) < tol
    g_dev = torch.autograd.grad((got.float() * dy.cuda()).sum(), dev)
    for i, (a, r) in enumerate(zip(g_dev, g_ref)):
        assert O.rel_l2(a.float().cpu(), r.float()) < tol, i
    # bit-reproducible, parameter gradients included
    q2, k2, v2 = dn.gdn_qkv_producer(dev[0], dev[1], dev[2] if with_bias else None, num_k_heads=Hk, num_v_heads=Hv,
                                     head_k_dim=K, head_v_dim=V, segment_ids=None if seg is None else seg.cuda())
    got2 = torch.cat([q2.reshape(B, L, -1), k2.reshape(B, L, -1), v2.reshape(B, L, -1)], -1)
    for a, b2 in zip(g_dev, torch.autograd.grad((got2.float() * dy.cuda()).sum(), dev)):
        assert torch.equal(a, b2)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
def test_gates(dn, dtype, tol):
    B, L, Hv = 2, 257, 6
    gen = torch.Generator().manual_seed(20)
    a, b = (torch.randn(B, L, Hv, generator=gen) * 2).to(dtype), (torch.randn(B, L, Hv, generator=gen) * 2).to(dtype)
    A_log, dt_bias = torch.log(1 + 15 * torch.rand(Hv, generator=gen)), torch.randn(Hv, generator=gen) * 0.5
    dg, dbeta = torch.randn(B, L, Hv, generator=gen), torch.randn(B, L, Hv, generator=gen)
    lv = [t.clone().requires_grad_() for t in (a, b, A_log, dt_bias)]
    g_ref = -lv[2].float().exp() * F.softplus(lv[0].float() + lv[3])
    beta_ref = lv[1].float().sigmoid()
    gr = torch.autograd.grad((g_ref * dg).sum() + (beta_ref * dbeta).sum(), lv)
    dv = [t.cuda().requires_grad_() for t in (a, b, A_log, dt_bias)]
    g, beta = dn.gdn_gates(*dv)
    assert g.dtype == torch.float32 and beta.dtype == torch.float32
    assert O.rel_l2(g.cpu(), g_ref.detach()) < 1e-5 and O.rel_l2(beta.cpu(), beta_ref.detach()) < 1e-5
    gg = torch.autograd.grad((g * dg.cuda()).sum() + (beta * dbeta.cuda()).sum(), dv)
    for i, (x, r) in enumerate(zip(gg, gr)):
        assert O.rel_l2(x.float().cpu(), r.float()) < tol, i


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("V", [128, 64])
def test_gated_rmsnorm_matches_qwen3_5_module(dn, dtype, tol, V):
    """Forward and all gradients against transformers' Qwen3_5RMSNormGated (a black-box reference)."""
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5RMSNormGated
    B, L, Hv = 2, 100, 3
    gen = torch.Generator().manual_seed(30 + V)
    o, z = (torch.randn(B, L, Hv, V, generator=gen) * 2).to(dtype), torch.randn(B, L, Hv, V, generator=gen).to(dtype)
    weight = 1 + 0.2 * torch.randn(V, generator=gen)
    dy = torch.randn(B, L, Hv, V, generator=gen).to(dtype).float()
    mod = Qwen3_5RMSNormGated(V, eps=1e-6)
    with torch.no_grad():
        mod.weight.copy_(weight)
    lo, lz = o.clone().requires_grad_(), z.clone().requires_grad_()
    y_ref = mod(lo.reshape(-1, V), lz.reshape(-1, V)).reshape(B, L, Hv, V)
    gr = torch.autograd.grad((y_ref.float() * dy).sum(), [lo, lz, mod.weight])
    do_, dz_, dw_ = o.cuda().requires_grad_(), z.cuda().requires_grad_(), weight.cuda().requires_grad_()
    y = dn.gated_rmsnorm(do_, dz_, dw_, eps=1e-6)
    assert y.shape == o.shape and y.dtype == dtype
    assert O.rel_l2(y.float().cpu(), y_ref.detach().float()) < tol
    gg = torch.autograd.grad((y.float() * dy.cuda()).sum(), [do_, dz_, dw_])
    for i, (x, r) in enumerate(zip(gg, gr)):
        assert O.rel_l2(x.float().cpu(), r.float()) < (tol if i < 2 else 2 * tol), i
    y2 = dn.gated_rmsnorm(do_, dz_, dw_, eps=1e-6)
    for a, b2 in zip(gg, torch.autograd.grad((y2.float() * dy.cuda()).sum(), [do_, dz_, dw_])):
        assert torch.equal(a, b2)


def test_layer_core_matches_qwen3_5_torch_reference(dn):
    """producer -> gates -> chunk_gdn -> gated norm on the GPU against the same chain built from
    transformers' torch_chunk_gated_delta_rule and plain torch ops on the CPU (fp32), Qwen3.5's head layout
    (Hk = 2, Hv = 4, K = V = 128, conv width 4)."""
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5RMSNormGated, torch_chunk_gated_delta_rule
    B, L, Hk, Hv, K, V, W = 1, 192, 2, 4, 128, 128, 4
    D = 2 * Hk * K + Hv * V
    gen = torch.Generator().manual_seed(40)
    mixed = torch.randn(B, L, D, generator=gen)
    w = torch.randn(D, 1, W, generator=gen) * 0.5
    a, b = torch.randn(B, L, Hv, generator=gen), torch.randn(B, L, Hv, generator=gen)
    A_log, dt_bias = torch.log(1 + 15 * torch.rand(Hv, generator=gen)), torch.randn(Hv, generator=gen) * 0.5
    z = torch.randn(B, L, Hv, V, generator=gen)
    nw = 1 + 0.2 * torch.randn(V, generator=gen)
    # CPU chain
    conv = conv_ref(mixed, w, None, None)
    q, k, v = torch.split(conv, [Hk * K, Hk * K, Hv * V], -1)
    q, k, v = q.reshape(B, L, Hk, K), k.reshape(B, L, Hk, K), v.reshape(B, L, Hv, V)
    beta = b.sigmoid()
    g = -A_log.exp() * F.softplus(a + dt_bias)
    o_ref, s_ref = torch_chunk_gated_delta_rule(q.repeat_interleave(Hv // Hk, 2), k.repeat_interleave(Hv // Hk, 2), v, g=g,
                                                beta=beta, initial_state=None, output_final_state=True,
                                                use_qk_l2norm_in_kernel=True)
    mod = Qwen3_5RMSNormGated(V, eps=1e-6)
    with torch.no_grad():
        mod.weight.copy_(nw)
        y_ref = mod(o_ref.reshape(-1, V), z.reshape(-1, V)).reshape(B, L, Hv * V)
    # GPU chain
    qd, kd, vd = dn.gdn_qkv_producer(mixed.cuda(), w.cuda(), None, num_k_heads=Hk, num_v_heads=Hv)
    gd, bd = dn.gdn_gates(a.cuda(), b.cuda(), A_log.cuda(), dt_bias.cuda())
    od, sd = dn.chunk_gdn(qd, kd, vd, gd, bd, output_final_state=True, is_inference=True, precision="fp32", qk_l2norm=True)
    yd = dn.gated_rmsnorm(od, z.cuda(), nw.cuda()).reshape(B, L, Hv * V)
    assert O.rel_l2(od.cpu(), o_ref) < 2e-4
    assert O.rel_l2(sd.cpu(), s_ref) < 2e-4
    assert O.rel_l2(yd.cpu(), y_ref) < 2e-4
