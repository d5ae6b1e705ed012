"""Process-group helpers with the reference's names (src/para_attn/primitives.py:14-148).

The hot-path exchange (head<->sequence all-to-all, K/V rotation) does not go through these:
it is done by the peer-store kernels of libpa_b200 (see ``_cp_engine``). What remains here
are the group accessors, the shard/unshard helpers called once per transformer forward, and
synchronous NCCL/gloo collectives for the small control-plane messages (seed agreement,
the two cache scalars, the exit all-gather).

Every ``group`` argument accepts ``None`` (the default group), a ``ProcessGroup`` or a
one-dimensional ``DeviceMesh``.
"""
from typing import Optional, Sequence, Union

import torch
import torch.distributed as dist
import torch.distributed._functional_collectives as funcol
from torch.distributed.distributed_c10d import _get_default_group

from . import config


# ------------------------------------------------------------------------------------------
# groups
# ------------------------------------------------------------------------------------------
def get_default_group() -> dist.ProcessGroup:
    return _get_default_group()


def get_group(group=None) -> dist.ProcessGroup:
    if isinstance(group, dist.ProcessGroup):
        return group
    return _get_default_group() if group is None else group.get_group()  # DeviceMesh -> its group


def get_world_size(group=None) -> int:
    return dist.get_world_size(get_group(group))


def get_rank(group=None) -> int:
    return dist.get_rank(get_group(group))


# ------------------------------------------------------------------------------------------
# collectives that return finished tensors (functional collectives hand out lazy ones)
# ------------------------------------------------------------------------------------------
def _finished(t: torch.Tensor) -> torch.Tensor:
    return t.wait() if isinstance(t, funcol.AsyncCollectiveTensor) else t


def all_gather_tensor_sync(x, *args, group=None, **kwargs):
    """All-gather along dim 0; works on the flattened tensor so that any trailing shape is kept."""
    lead, rest = x.shape[0], tuple(x.shape[1:])
    flat = x.flatten()
    gathered = _finished(funcol.all_gather_tensor(flat, *args, group=get_group(group), **kwargs))
    copies = gathered.numel() // max(flat.numel(), 1)
    return gathered.reshape((lead * copies,) + rest)


def all_to_all_single_sync(x, *args, **kwargs):
    """Equal-split all-to-all along the flattened tensor, reshaped back (used by callers that
    keep the reference's exchange; the fused attention path does not call it)."""
    return _finished(funcol.all_to_all_single(x.flatten(), *args, **kwargs)).reshape(x.shape)


def all_reduce_sync(x, *args, group=None, **kwargs):
    """``funcol.all_reduce`` that returns a finished tensor (src/para_attn/primitives.py:90-94).
    The gloo backend has no "avg" reduction: there the average is the fp32 sum divided by the
    group size and rounded back to the tensor's dtype (NCCL groups use NCCL's own "avg")."""
    pg = get_group(group)
    op = args[0] if args else kwargs.get("reduceOp")
    if isinstance(op, str) and op.lower() == "avg" and dist.get_backend(pg) == "gloo":
        total = _finished(funcol.all_reduce(x.float(), "sum", group=pg))
        return (total / dist.get_world_size(pg)).to(x.dtype)
    return _finished(funcol.all_reduce(x, *args, group=pg, **kwargs))


# ------------------------------------------------------------------------------------------
# sharding helpers
# ------------------------------------------------------------------------------------------
def get_buffer(shape_or_tensor: Union[Sequence[int], torch.Tensor], *, repeats: int = 1, dim: int = 0,
               dtype: Optional[torch.dtype] = None, device: Optional[torch.device] = None, group=None) -> torch.Tensor:
    """An uninitialised tensor shaped like ``shape_or_tensor`` with ``dim`` enlarged ``repeats``
    times (``repeats=None``: once per rank of ``group``) - a receive buffer for gathers."""
    if isinstance(shape_or_tensor, torch.Tensor):
        like = shape_or_tensor
        shape, dtype, device = list(like.shape), like.dtype, like.device
    else:
        shape = list(shape_or_tensor)
    assert dtype is not None
    assert device is not None
    factor = get_world_size(group) if repeats is None else repeats
    if factor > 1:
        shape[dim] = shape[dim] * factor
    return torch.empty(shape, dtype=dtype, device=device)


def get_assigned_chunk(tensor: torch.Tensor, dim: int = 0, idx: Optional[int] = None, group=None) -> torch.Tensor:
    """This rank's (or rank ``idx``'s) equal share of ``tensor`` along ``dim``; uneven splits are refused."""
    world_size = get_world_size(group)
    total_size = tensor.shape[dim]
    assert total_size % world_size == 0, f"tensor.shape[{dim}]={total_size} is not divisible by world_size={world_size}"
    which = get_rank(group) if idx is None else idx
    return tensor.chunk(world_size, dim=dim)[which]


def get_complete_tensor(tensor: torch.Tensor, *, dim: int = 0, group=None) -> torch.Tensor:
    """Inverse of ``get_assigned_chunk``: the shards of all ranks concatenated along ``dim``
    (src/para_attn/primitives.py:139-148). CUDA tensors on an NCCL group of up to eight ranks go
    through peer stores into every rank's result buffer (``_peer_gather``; switch off with
    ``config.cp.peer_gather``); everything else takes the transpose -> all_gather -> transpose of
    the reference."""
    pg = get_group(group)
    if (tensor.device.type == "cuda" and get_world_size(pg) > 1 and config.cp.peer_gather
            and dist.get_backend(pg) == "nccl" and get_world_size(pg) <= 8 and tensor.numel() > 0):
        from . import _peer_gather

        out = _peer_gather.get_gather(pg, tensor.device).gather(tensor, dim)
        if out is not None:
            return out
    moved = tensor.transpose(0, dim).contiguous()  # the gather concatenates along dim 0
    return all_gather_tensor_sync(moved, gather_dim=0, group=group).transpose(0, dim)
