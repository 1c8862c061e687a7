"""Argument validation of the public operators: the error messages the reference's own suite matches
(tests/test_validation.py:10-277 of the reference), raised before anything touches a device, so these
run on CPU tensors.  Where this build accepts a superset (chunk_size 64, K or V = 64) the rejected
value is one neither accepts."""
import pytest
import torch

import deltanet_b200 as dn


def base(B=1, L=128, Hk=2, Hv=4, K=128, V=128):
    z = torch.zeros
    return dict(q=z(B, L, Hk, K), k=z(B, L, Hk, K), v=z(B, L, Hv, V), g=z(B, L, Hk, K), b=z(B, L, Hk, K), w=z(B, L, Hv, V))


def call(t, **kw):
    return dn.chunk_gdn2(t["q"], t["k"], t["v"], t["g"], t["b"], t["w"], **kw)


def test_invalid_precision():
    with pytest.raises(ValueError, match="Invalid precision"):
        call(base(), precision="invalid_precision")


def test_precision_none_raises():
    with pytest.raises(ValueError, match="precision must be a string"):
        call(base(), precision=None)


def test_unsupported_chunk_size():
    with pytest.raises(ValueError, match="Unsupported chunk_size"):
        call(base(), chunk_size=32)


def test_unsupported_head_dims():
    with pytest.raises(ValueError, match="Unsupported head dimensions"):
        call(base(K=32, V=32))


def test_unsupported_head_ratio():
    t = base(Hk=3)
    with pytest.raises(ValueError, match="Value heads .* must be divisible by key heads"):
        call(t)


def test_invalid_cu_seqlens():
    with pytest.raises(ValueError, match="cu_seqlens.* must equal sequence length"):
        call(base(), cu_seqlens=[0, 64, 100])
    with pytest.raises(ValueError, match="strictly monotonically increasing"):
        call(base(), cu_seqlens=[0, 64, 32, 128])
    with pytest.raises(ValueError, match=r"cu_seqlens\[0\] must be 0"):
        call(base(), cu_seqlens=[1, 64, 128])
    with pytest.raises(ValueError, match="Cannot pass both segment_ids and cu_seqlens"):
        call(base(), cu_seqlens=[0, 128], segment_ids=torch.zeros(128, dtype=torch.int32))


def test_wrong_k_and_v_shapes():
    t = base()
    t["k"] = torch.zeros(1, 128, 3, 128)
    with pytest.raises(ValueError, match="Key tensor k shape"):
        call(t)
    t = base()
    t["v"] = torch.zeros(1, 64, 4, 128)
    with pytest.raises(ValueError, match="Value tensor v shape"):
        call(t)
    t = base()
    t["q"] = torch.zeros(128, 2, 128)
    with pytest.raises(ValueError, match="Query tensor q must be 4D"):
        call(t)


@pytest.mark.parametrize("name", ["g", "b", "w"])
def test_wrong_gate_shapes(name):
    t = base()
    t[name] = torch.zeros(1, 128, t[name].shape[2], 64)
    with pytest.raises(ValueError, match=f"{name} last dimension"):
        call(t)
    t = base()
    t[name] = torch.zeros(1, 128, 3, 128)
    with pytest.raises(ValueError, match=f"{name} head dimension"):
        call(t)
    t = base()
    t[name] = torch.zeros(1, 128)
    with pytest.raises(ValueError, match=f"{name} must have rank 3"):
        call(t)


def test_segment_ids_checks():
    with pytest.raises(ValueError, match="segment_ids length"):
        call(base(), segment_ids=torch.zeros(64, dtype=torch.int32))
    with pytest.raises(ValueError, match="segment_ids must have integer dtype"):
        call(base(), segment_ids=torch.zeros(1, 128, dtype=torch.float32))
    with pytest.raises(ValueError, match="2D segment_ids shape"):
        call(base(), segment_ids=torch.zeros(2, 128, dtype=torch.int32))


def test_initial_state_shape_mismatch():
    with pytest.raises(ValueError, match="initial_state shape"):
        call(base(), initial_state=torch.zeros(1, 2, 128, 128))


def test_fuse_prologue_requires_l2norm():
    with pytest.raises(ValueError, match="fuse_prologue=True requires qk_l2norm=True"):
        call(base(), fuse_prologue=True)


def test_scale_must_be_concrete():
    with pytest.raises(ValueError, match="scale must be a concrete Python float or scalar"):
        call(base(), scale=torch.ones(2))
    with pytest.raises(ValueError, match="scale must be convertible to a concrete float"):
        call(base(), scale="big")


def test_nonpositive_stability_tau_and_block_size_raise():
    with pytest.raises(ValueError, match="stability_tau"):
        call(base(), stability_guard=True, stability_tau=-1.0)
    with pytest.raises(ValueError, match="prefill_block_size"):
        call(base(), is_inference=True, streaming_prefill=True, prefill_block_size=0)
    t = base()
    state = torch.zeros(1, 4, 128, 128)
    with pytest.raises(ValueError, match="stability_tau"):
        dn.gdn2_decode_step(t["q"][:, 0], t["k"][:, 0], t["v"][:, 0], t["g"][:, 0], t["b"][:, 0], t["w"][:, 0], state,
                            stability_guard=True, stability_tau=0.0)


def test_decode_step_validation():
    z = torch.zeros
    q, k, v, g, b, w = z(1, 2, 128), z(1, 2, 128), z(1, 4, 128), z(1, 2, 128), z(1, 2, 128), z(1, 4, 128)
    state = z(1, 4, 128, 128)
    with pytest.raises(ValueError, match="state shape"):
        dn.gdn2_decode_step(q, k, v, g, b, w, z(1, 2, 128, 128))
    with pytest.raises(ValueError, match="Key tensor k shape"):
        dn.gdn2_decode_step(q, z(1, 3, 128), v, g, b, w, state)
    with pytest.raises(ValueError, match="Value tensor v batch"):
        dn.gdn2_decode_step(q, k, z(2, 4, 128), g, b, w, state)
    with pytest.raises(ValueError, match="Decode step sequence dimension must be 1"):
        dn.gdn2_decode_step(z(1, 2, 2, 128), z(1, 2, 2, 128), z(1, 2, 4, 128), g, b, w, state)


def test_decode_reset_shape_raises():
    z = torch.zeros
    q, k, v, g, b, w = z(2, 2, 128), z(2, 2, 128), z(2, 4, 128), z(2, 2, 128), z(2, 2, 128), z(2, 4, 128)
    with pytest.raises(ValueError, match="reset batch dimension"):
        dn.gdn2_decode_step(q, k, v, g, b, w, z(2, 4, 128, 128), reset=torch.tensor([True]))


def test_channel_wise_beta_in_variants_raises():
    t = base()
    beta_cw = torch.zeros(1, 128, 2, 128)
    with pytest.raises(ValueError, match="channel-wise beta with shape"):
        dn.chunk_gdn(t["q"], t["k"], t["v"], t["g"][..., :1], beta_cw)
    with pytest.raises(ValueError, match="channel-wise beta with shape"):
        dn.chunk_kda(t["q"], t["k"], t["v"], t["g"], beta_cw)
    with pytest.raises(ValueError, match="channel-wise beta with shape"):
        dn.chunk_delta_rule(t["q"], t["k"], t["v"], beta_cw)
    z = torch.zeros
    with pytest.raises(ValueError, match="channel-wise beta with shape"):
        dn.gdn_decode_step(z(1, 2, 128), z(1, 2, 128), z(1, 4, 128), z(1, 4), z(1, 2, 128), z(1, 4, 128, 128))


def test_valid_arguments_reach_the_device_check():
    """Valid arguments pass validation and stop at the one thing a CPU box cannot do."""
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        call(base())
