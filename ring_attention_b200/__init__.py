"""B200-native ring attention behind the API of jondeaton/ring-attention-jax-pallas.

`ring_attention` and `ring_self_attention` are what ring_attention/__init__.py:3 of the
reference re-exports; the rest is the host plumbing a one-process-per-GPU program needs.
"""
from ._lib import LIB_PATH, RingAttentionError, device_status
from .layout import zigzag_indices, zigzag_shard, zigzag_unshard
from .mesh import Mesh, PartitionSpec, Ring
from .ring import RingPlan, ScoreMod, bwd_block, fwd_block, make_ring_plan, reserve, ring_attention, ring_self_attention

__all__ = [
    "ring_attention", "ring_self_attention", "fwd_block", "bwd_block", "ScoreMod",
    "Mesh", "PartitionSpec", "Ring", "RingAttentionError", "LIB_PATH",
    "zigzag_indices", "zigzag_shard", "zigzag_unshard", "RingPlan", "make_ring_plan", "device_status", "reserve",
]
