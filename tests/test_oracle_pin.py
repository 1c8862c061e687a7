"""The CPU oracle against two independent third-party recurrences (used as black boxes).

The reference's own example validates its GDN path against transformers' Qwen3.5 torch
implementation (examples/qwen3_5_layer_parity.py:135-168 of the reference); the same
comparison is made here for the oracle, plus flash-linear-attention's naive KDA recurrence.
"""
import warnings

import pytest
import torch

from oracle import delta_oracle as O


def test_against_transformers_gated_delta_rule():
    m = pytest.importorskip("transformers.models.qwen3_5.modeling_qwen3_5")
    torch.manual_seed(0)
    B, L, H, K, V = 1, 192, 2, 64, 64
    q, k, v = torch.randn(B, L, H, K), torch.randn(B, L, H, K), torch.randn(B, L, H, V)
    g = -torch.exp(torch.randn(B, L, H) * 0.39 - 1.0)
    beta = torch.sigmoid(torch.randn(B, L, H))
    ref_o, ref_s = m.torch_recurrent_gated_delta_rule(q, k, v, g, beta, initial_state=None,
                                                     output_final_state=True, use_qk_l2norm_in_kernel=True)
    o, s = O.token_serial_gdn2(q, k, v, g, beta, beta, qk_l2norm=True, output_final_state=True)
    assert O.rel_l2(o, ref_o) < 1e-5
    assert O.rel_l2(s, ref_s) < 1e-5
    o2, s2 = O.chunk_gdn(q, k, v, g, beta, qk_l2norm=True, output_final_state=True, chunk_size=64,
                         precision="fp32")
    assert O.rel_l2(o2, ref_o) < 1e-5
    assert O.rel_l2(s2, ref_s) < 1e-5


def test_against_fla_naive_kda():
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        naive = pytest.importorskip("fla.ops.kda.naive")
    torch.manual_seed(1)
    B, L, H, K, V = 1, 128, 2, 64, 64
    q, k, v = torch.randn(B, L, H, K), torch.randn(B, L, H, K), torch.randn(B, L, H, V)
    k = k / k.norm(dim=-1, keepdim=True)
    g = -torch.exp(torch.randn(B, L, H, K) * 0.39 - 1.0)
    beta = torch.sigmoid(torch.randn(B, L, H))
    ref_o, ref_s = naive.naive_recurrent_kda(q, k, v, g, beta, output_final_state=True)
    o, s = O.token_serial_gdn2(q, k, v, g, beta, beta, output_final_state=True)
    assert O.rel_l2(o, ref_o) < 1e-5
    assert O.rel_l2(s, ref_s) < 1e-5
