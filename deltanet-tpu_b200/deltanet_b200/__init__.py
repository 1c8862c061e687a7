"""deltanet_b200: the delta-rule recurrence core of deltanet-tpu on B200 (sm_100a).

Public names are the reference's (``src/deltanet_tpu/__init__.py:3-29``).
"""
from .gdn2 import chunk_gdn2, gdn2_decode_step
from .layer_steps import gated_rmsnorm, gdn_gates, gdn_qkv_producer
from .variants import (
    chunk_delta_rule,
    chunk_gdn,
    chunk_gla,
    chunk_kda,
    delta_rule_decode_step,
    gdn_decode_step,
    gla_decode_step,
    kda_decode_step,
)

__all__ = [
    "chunk_gdn2", "gdn2_decode_step", "chunk_gdn", "chunk_kda", "chunk_gla", "chunk_delta_rule",
    "gdn_decode_step", "kda_decode_step", "gla_decode_step", "delta_rule_decode_step",
    "gdn_qkv_producer", "gdn_gates", "gated_rmsnorm",
]
__version__ = "0.1.0"
