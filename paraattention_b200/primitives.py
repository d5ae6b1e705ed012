"""Process-group helpers with the reference's names (src/para_attn/primitives.py:14-148).

The hot-path exchange (head<->sequence all-to-all, K/V rotation) does not go through these:
it is done by the peer-store kernels of libpa_b200 (see ``_cp_engine``). What remains here
are the group accessors, the shard/unshard helpers called once per transformer forward, and
synchronous NCCL/gloo collectives for the small control-plane messages (seed agreement,
the two cache scalars, the exit all-gather).
"""
from typing import List, Optional, Tuple, Union

import torch
import torch.distributed as dist
import torch.distributed._functional_collectives as ft_c
import torch.distributed.distributed_c10d as c10d


def get_default_group():
    return c10d._get_default_group()


def get_group(group=None):
    if group is None:
        group = c10d._get_default_group()
    if isinstance(group, dist.ProcessGroup):
        return group
    return group.get_group()


def get_world_size(group=None):
    return dist.get_world_size(get_group(group))


def get_rank(group=None):
    return dist.get_rank(get_group(group))


def _maybe_wait(tensor: torch.Tensor) -> torch.Tensor:
    if isinstance(tensor, ft_c.AsyncCollectiveTensor):
        return tensor.wait()
    return tensor


def all_gather_tensor_sync(x, *args, group=None, **kwargs):
    group = get_group(group)
    x_shape = list(x.shape)
    x = x.flatten()
    x_numel = x.numel()
    x = _maybe_wait(ft_c.all_gather_tensor(x, *args, group=group, **kwargs))
    x_shape[0] *= x.numel() // x_numel
    return x.reshape(x_shape)


def all_to_all_single_sync(x, *args, **kwargs):
    x_shape = x.shape
    x = _maybe_wait(ft_c.all_to_all_single(x.flatten(), *args, **kwargs))
    return x.reshape(x_shape)


def all_reduce_sync(x, *args, group=None, **kwargs):
    group = get_group(group)
    return _maybe_wait(ft_c.all_reduce(x, *args, group=group, **kwargs))


def get_buffer(
    shape_or_tensor: Union[Tuple[int], torch.Tensor],
    *,
    repeats: int = 1,
    dim: int = 0,
    dtype: Optional[torch.dtype] = None,
    device: Optional[torch.device] = None,
    group=None,
) -> torch.Tensor:
    if repeats is None:
        repeats = get_world_size(group)
    if isinstance(shape_or_tensor, torch.Tensor):
        shape, dtype, device = shape_or_tensor.shape, shape_or_tensor.dtype, shape_or_tensor.device
    else:
        shape = shape_or_tensor
    assert dtype is not None
    assert device is not None
    shape = list(shape)
    if repeats > 1:
        shape[dim] *= repeats
    return torch.empty(shape, dtype=dtype, device=device)


def get_assigned_chunk(tensor: torch.Tensor, dim: int = 0, idx: Optional[int] = None, group=None) -> torch.Tensor:
    if idx is None:
        idx = get_rank(group)
    world_size = get_world_size(group)
    total_size = tensor.shape[dim]
    assert total_size % world_size == 0, f"tensor.shape[{dim}]={total_size} is not divisible by world_size={world_size}"
    return tensor.chunk(world_size, dim=dim)[idx]


def get_complete_tensor(tensor: torch.Tensor, *, dim: int = 0, group=None) -> torch.Tensor:
    tensor = tensor.transpose(0, dim).contiguous()
    output_tensor = all_gather_tensor_sync(tensor, gather_dim=0, group=group)
    return output_tensor.transpose(0, dim)
