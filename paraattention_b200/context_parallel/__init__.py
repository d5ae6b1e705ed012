"""Device-mesh construction for context parallelism (src/para_attn/context_parallel/__init__.py:8-39).

The mesh has three named dimensions, ("batch", "ring", "ulysses"), with "ulysses" varying
fastest: neighbouring ranks form a Ulysses group, which is also the order in which the fused
exchange numbers the sequence chunks (flat rank = ring index * ulysses size + ulysses index).
"""
import math
from typing import Optional, Tuple

import torch.distributed as dist

from .. import primitives as DP

MESH_DIM_NAMES = ("batch", "ring", "ulysses")


def _largest_common_factor(total: int, limit: Optional[int]) -> int:
    """gcd(total, limit): the largest size <= limit that divides the ranks evenly; 1 without a limit."""
    return math.gcd(total, limit) if limit is not None else 1


def mesh_shape_for(world_size: int, max_batch_dim_size: Optional[int] = None, max_ring_dim_size: Optional[int] = None,
                   max_ulysses_dim_size: Optional[int] = None) -> Tuple[int, int, int]:
    """(batch, ring, ulysses) sizes. Ranks go to "batch" first (classifier-free-guidance pairs), the
    rest is attention parallelism: all Ulysses by default, with one of the two limits deciding the
    split between ring and Ulysses."""
    assert max_ring_dim_size is None or max_ulysses_dim_size is None, \
        "Only one of max_ulysses_dim_size and max_ring_dim_size can be set"
    batch = _largest_common_factor(world_size, max_batch_dim_size)
    attention_ranks = world_size // batch
    if max_ulysses_dim_size is not None:
        ulysses = math.gcd(attention_ranks, max_ulysses_dim_size)
        return batch, attention_ranks // ulysses, ulysses
    ring = _largest_common_factor(attention_ranks, max_ring_dim_size)
    return batch, ring, attention_ranks // ring


def init_context_parallel_mesh(device_type=None, *, mesh=None, max_batch_dim_size=None, max_ring_dim_size=None,
                               max_ulysses_dim_size=None):
    if mesh is not None:
        return mesh
    assert device_type is not None, "device must be provided if mesh is not provided"
    shape = mesh_shape_for(DP.get_world_size(), max_batch_dim_size, max_ring_dim_size, max_ulysses_dim_size)
    return dist.init_device_mesh(device_type, shape, mesh_dim_names=MESH_DIM_NAMES)
