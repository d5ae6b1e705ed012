"""Ring / Ulysses / unified context-parallel attention with the reference's interface
(src/para_attn/para_attn_interface.py): ``ring_attn_func``, ``ulysses_attn_func``,
``in_batch_attn_func`` and the TorchFunctionModes ``RingAttnMode``, ``UlyssesAttnMode``,
``UnifiedAttnMode``, ``InBatchAttnMode`` that intercept ``F.scaled_dot_product_attention``.

Same signatures, assertions and results; what runs underneath differs. With more than one
rank an attention call becomes a peer-store exchange plus ONE chunked tcgen05 attention
launch per rank (``_cp_engine``) instead of NCCL all-to-alls around per-step SDPA calls and
an fp32 merge; with one rank it is the plain sm_100a attention kernel (``ops``).
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import _cp_engine
from . import ops as para_attn_ops
from . import primitives as DP
from .utils import base_handle_torch_function, BaseTorchFunctionMode, get_allow_sdpa_fallback

__all__ = [
    "UnifiedAttnMode",
    "RingAttnMode",
    "UlyssesAttnMode",
    "InBatchAttnMode",
    "ring_attn_func",
    "ulysses_attn_func",
    "in_batch_attn_func",
    "unified_attn_func",
    "sparse_kv_attn_func",
    "SparseKVAttnMode",
]


def _kernel_can_run(query, key, value, attn_mask, dropout_p, is_causal, total_keys=None) -> bool:
    """Whether the sm_100a kernel covers this call. A mask is covered when it is a boolean
    key-padding mask over ``total_keys`` keys (default: the keys of ``key``) and the call is not causal."""
    if attn_mask is not None:
        if query.ndim != 4 or is_causal:
            return False
        n = key.shape[-2] if total_keys is None else total_keys
        if para_attn_ops.key_mask_of(attn_mask, query.shape[0], n) is None:
            return False
    return (
        query.device.type == "cuda"
        and query.dtype in (torch.bfloat16, torch.float16)
        and key.dtype == query.dtype
        and value.dtype == query.dtype
        and query.ndim == 4
        and query.shape[-1] in (64, 128)
        and key.shape[-1] == query.shape[-1]
        and value.shape[-1] == query.shape[-1]
        and dropout_p == 0.0
    )


def _local_attention(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *, scale=None):
    """The non-parallel SDPA at the bottom of every mode (state "none" of the reference,
    src/para_attn/para_attn_interface.py:468-475): the sm_100a kernel. A call the kernel does
    not cover (CPU tensors, fp32, another head_dim, a general mask, dropout) raises; only with
    ``config.attention.allow_sdpa_fallback`` set is it handed to PyTorch's own SDPA instead."""
    if _kernel_can_run(query, key, value, attn_mask, dropout_p, is_causal):
        if attn_mask is not None:
            return para_attn_ops.attention_forward_sparse_kv(query, key, value, attn_mask=attn_mask, scale=scale)
        return para_attn_ops.attention_forward(query, key, value, is_causal=is_causal, scale=scale)
    if get_allow_sdpa_fallback():
        return F.scaled_dot_product_attention(
            query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal, scale=scale)
    raise NotImplementedError(
        "attention outside the sm_100a kernel's coverage (CUDA bf16/f16, head_dim 64 or 128, no dropout, no mask other "
        f"than a boolean key-padding mask): got {query.device.type} {query.dtype} head_dim {query.shape[-1]}"
        f"{', a mask' if attn_mask is not None else ''}{', dropout' if dropout_p else ''}. "
        "Set paraattention_b200.config.attention.allow_sdpa_fallback = True to let PyTorch's SDPA take such calls.")


@torch.compiler.assume_constant_result
def _engine_id(flat_group, ulysses, ring, u, r, device_index):
    return _cp_engine.engine_id(flat_group, ulysses, ring, u, r, device_index)


def _cp_attention(query, key, value, scale, *, flat_group, ulysses, ring, u, r, is_causal=False, attn_mask=None):
    # (CPU tensors never get here: _require_kernel refuses them, and the op below is CUDA-only)
    eid = _engine_id(flat_group, ulysses, ring, u, r, query.device.index)
    key_mask = None
    if attn_mask is not None:
        # keys of all ranks, chunk by chunk in flat-rank order: for a Ulysses group that is the
        # order its all-to-all produces (src/para_attn/para_attn_interface.py:60-72), the layout
        # the reference's adapters build their masks in
        key_mask = para_attn_ops.key_mask_of(attn_mask, query.shape[0], ulysses * ring * key.shape[2])
    return para_attn_ops.cp_attention_forward(query, key, value, key_mask, bool(is_causal), scale, eid)


def _require_kernel(query, key, value, attn_mask, dropout_p, is_causal, what, world=1):
    if not _kernel_can_run(query, key, value, attn_mask, dropout_p, is_causal, total_keys=world * key.shape[-2]):
        raise NotImplementedError(
            f"{what}: the context-parallel kernel is built for CUDA bf16/f16 tensors with head_dim 64 or 128, "
            "no dropout, and no mask other than a boolean key-padding mask [B, 1, 1, keys of all ranks] "
            "(not together with is_causal)")


def ulysses_attn_func(
    query,
    key,
    value,
    attn_mask=None,
    dropout_p=0.0,
    is_causal=False,
    *,
    scale=None,
    mesh=None,
    attn_func=None,
):
    assert query.ndim == 4, "query must have 4 dimensions, got {}".format(query.ndim)
    assert key.ndim == 4, "key must have 4 dimensions, got {}".format(key.ndim)
    assert value.ndim == 4, "value must have 4 dimensions, got {}".format(value.ndim)

    pg = DP.get_group(mesh)
    world_size = DP.get_world_size(pg)
    if world_size <= 1:
        if attn_func is None:
            attn_func = _local_attention
        return attn_func(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal, scale=scale)

    h = query.shape[1]
    assert h % world_size == 0, "h must be divisible by world_size, got {} and {}".format(h, world_size)
    if attn_func is not None and attn_func is not F.scaled_dot_product_attention:
        raise NotImplementedError(
            "ulysses_attn_func with a custom attn_func: the head<->sequence exchange is fused into the attention "
            "kernel and cannot wrap a foreign attention function")
    _require_kernel(query, key, value, attn_mask, dropout_p, is_causal, "ulysses_attn_func", world_size)
    return _cp_attention(query, key, value, scale, flat_group=pg, ulysses=world_size, ring=1,
                         u=DP.get_rank(pg), r=0, is_causal=is_causal, attn_mask=attn_mask)


def ring_attn_func(
    query,
    key,
    value,
    attn_mask=None,
    dropout_p=0.0,
    is_causal=False,
    *,
    scale=None,
    mesh=None,
):
    pg = DP.get_group(mesh)
    world_size = DP.get_world_size(pg)
    if world_size <= 1:
        return _local_attention(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal,
                                scale=scale)

    # The reference asserts attn_mask is None here (src/para_attn/para_attn_interface.py:228); a
    # boolean key-padding mask over the keys of all ranks is the one kind that is accepted.
    assert attn_mask is None or (query.ndim == 4 and para_attn_ops.key_mask_of(
        attn_mask, query.shape[0], world_size * key.shape[-2]) is not None), \
        "attn_mask is not supported in ring_attn_func when world_size > 1"
    _require_kernel(query, key, value, attn_mask, dropout_p, is_causal, "ring_attn_func", world_size)
    return _cp_attention(query, key, value, scale, flat_group=pg, ulysses=1, ring=world_size, u=0,
                         r=DP.get_rank(pg), is_causal=is_causal, attn_mask=attn_mask)


def unified_attn_func(
    query,
    key,
    value,
    attn_mask=None,
    dropout_p=0.0,
    is_causal=False,
    *,
    scale=None,
    ulysses_mesh=None,
    ring_mesh=None,
    flat_group=None,
):
    """Ulysses outside, ring inside (what UnifiedAttnMode composes at
    src/para_attn/para_attn_interface.py:445-467) as one fused exchange + attention."""
    U = DP.get_world_size(ulysses_mesh) if ulysses_mesh is not None else 1
    R = DP.get_world_size(ring_mesh) if ring_mesh is not None else 1
    if U * R <= 1:
        return _local_attention(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal,
                                scale=scale)
    if R <= 1:
        return ulysses_attn_func(query, key, value, attn_mask, dropout_p, is_causal, scale=scale, mesh=ulysses_mesh)
    if U <= 1:
        return ring_attn_func(query, key, value, attn_mask, dropout_p, is_causal, scale=scale, mesh=ring_mesh)
    assert query.ndim == 4, "query must have 4 dimensions, got {}".format(query.ndim)
    assert query.shape[1] % U == 0, "h must be divisible by world_size, got {} and {}".format(query.shape[1], U)
    assert attn_mask is None or para_attn_ops.key_mask_of(
        attn_mask, query.shape[0], U * R * key.shape[-2]) is not None, \
        "attn_mask is not supported in ring_attn_func when world_size > 1"
    assert flat_group is not None, "a process group spanning the ulysses x ring ranks is required"
    _require_kernel(query, key, value, attn_mask, dropout_p, is_causal, "unified attention", U * R)
    return _cp_attention(query, key, value, scale, flat_group=flat_group, ulysses=U, ring=R,
                         u=DP.get_rank(ulysses_mesh), r=DP.get_rank(ring_mesh), is_causal=is_causal,
                         attn_mask=attn_mask)


def in_batch_attn_func(
    query,
    key,
    value,
    attn_mask=None,
    dropout_p=0.0,
    is_causal=False,
    *,
    scale=None,
):
    """Every batch element attends to the keys of ALL batch elements
    (src/para_attn/para_attn_interface.py:242-276): the batch is folded into the sequence, one
    attention runs over [1, H, B*S, D], and the result is unfolded again."""
    for name, t in (("query", query), ("key", key), ("value", value)):
        assert t.ndim == 4, "{} must have 4 dimensions, got {}".format(name, t.ndim)
    assert attn_mask is None, "attn_mask is not supported in in_batch_attn_func"
    assert not is_causal, "is_causal is not supported in in_batch_attn_func"

    batch, heads, s_q = query.shape[:3]

    def fold(t):  # [B, H, S, D] -> [1, H, B*S, D]
        return t.transpose(0, 1).reshape(1, heads, batch * t.shape[2], t.shape[3])

    folded = _local_attention(fold(query), fold(key), fold(value), dropout_p=dropout_p, scale=scale)
    return folded.reshape(heads, batch, s_q, folded.shape[-1]).transpose(0, 1)


def _get_arg(args, kwargs, *field):
    if len(field) == 1:
        return kwargs.get(field[0])
    index, name = field
    if index < len(args):
        return args[index]
    return kwargs.get(name)


def _get_args(args, kwargs, *names):
    return [_get_arg(args, kwargs, i, name) for i, name in enumerate(names)]


class _AttnModeBase(BaseTorchFunctionMode):
    """Shared plumbing: class-level ``disabled`` switch with a ``disable()`` context manager and
    the ``skip_small_kv`` bypass (src/para_attn/para_attn_interface.py:303-345)."""

    disabled = False

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = {} if kwargs is None else kwargs
        if type(self).disabled:
            return base_handle_torch_function(func, types, args, kwargs)
        if func is F.scaled_dot_product_attention:
            if self._skip_small_kv:
                query, key = _get_args(args, kwargs, "query", "key")
                if query.shape[-2] > key.shape[-2]:
                    return base_handle_torch_function(func, types, args, kwargs)
            return self._call_attn_func(*args, **kwargs)
        return base_handle_torch_function(func, types, args, kwargs)

    @classmethod
    @contextlib.contextmanager
    def disable(cls):
        old_disabled = cls._set_disabled(True)
        try:
            yield
        finally:
            cls._set_disabled(old_disabled)

    @classmethod
    @torch.compiler.disable
    def _set_disabled(cls, value):
        old_disabled = cls.disabled
        cls.disabled = value
        return old_disabled


class RingAttnMode(_AttnModeBase):
    disabled = False

    @torch.compiler.disable
    def __init__(self, mesh=None, *, skip_small_kv=False):
        super().__init__()
        self._mesh = mesh
        self._skip_small_kv = skip_small_kv

    def _call_attn_func(self, *args, **kwargs):
        return ring_attn_func(*args, **kwargs, mesh=self._mesh)

    _call_ring_attn_func = _call_attn_func


class UlyssesAttnMode(_AttnModeBase):
    disabled = False

    @torch.compiler.disable
    def __init__(self, mesh=None, *, attn_func=None, skip_small_kv=False):
        super().__init__()
        self._mesh = mesh
        self._attn_func = attn_func
        self._skip_small_kv = skip_small_kv

    def _call_attn_func(self, *args, **kwargs):
        return ulysses_attn_func(*args, **kwargs, mesh=self._mesh, attn_func=self._attn_func)

    _call_ulysses_attn_func = _call_attn_func


def _flat_group_of(mesh):
    """Process group over all ranks of the ("ring", "ulysses") sub-mesh of this rank."""
    names = [n for n in ("ring", "ulysses") if n in mesh.mesh_dim_names]
    sub = mesh[tuple(names)] if len(names) > 1 else mesh[names[0]]
    if sub.ndim == 1:
        return sub.get_group()
    return sub._flatten().get_group()


class UnifiedAttnMode(_AttnModeBase):
    disabled = False

    @torch.compiler.disable
    def __init__(self, mesh=None, *, skip_small_kv=False, attn_func=None):
        super().__init__()

        self._flat_group = None
        if mesh is None:
            self._ulysses_mesh = DP.get_default_group()
            self._ring_mesh = None
        else:
            if isinstance(mesh, dist.ProcessGroup):
                self._ulysses_mesh = mesh
                self._ring_mesh = None
            else:
                assert isinstance(mesh, dist.DeviceMesh), "mesh must be a ProcessGroup or DeviceMesh"

                if "ulysses" in mesh.mesh_dim_names:
                    self._ulysses_mesh = mesh["ulysses"]
                else:
                    self._ulysses_mesh = None
                if "ring" in mesh.mesh_dim_names:
                    self._ring_mesh = mesh["ring"]
                else:
                    self._ring_mesh = None

                assert (
                    self._ulysses_mesh is not None or self._ring_mesh is not None
                ), "mesh must have ulysses or ring dim"
                if self._ulysses_mesh is not None and self._ring_mesh is not None:
                    if self._ulysses_mesh.size() > 1 and self._ring_mesh.size() > 1:
                        self._flat_group = _flat_group_of(mesh)

        self._skip_small_kv = skip_small_kv
        self._attn_func = attn_func

    def _call_attn_func(self, *args, **kwargs):
        query, key, value, attn_mask, dropout_p, is_causal = _get_args(
            args, kwargs, "query", "key", "value", "attn_mask", "dropout_p", "is_causal")
        scale = kwargs.get("scale")
        dropout_p = 0.0 if dropout_p is None else dropout_p
        is_causal = False if is_causal is None else is_causal
        U = DP.get_world_size(self._ulysses_mesh) if self._ulysses_mesh is not None else 1
        R = DP.get_world_size(self._ring_mesh) if self._ring_mesh is not None else 1
        if self._attn_func is not None and self._attn_func is not F.scaled_dot_product_attention:
            if U * R <= 1:
                return self._attn_func(*args, **kwargs)
            raise NotImplementedError(
                "UnifiedAttnMode with a custom attn_func on a parallel mesh: the exchange is fused into the attention "
                "kernel and cannot wrap a foreign attention function")
        return unified_attn_func(query, key, value, attn_mask, dropout_p, is_causal, scale=scale,
                                 ulysses_mesh=self._ulysses_mesh, ring_mesh=self._ring_mesh,
                                 flat_group=self._flat_group)

    _call_unified_attn_func = _call_attn_func


def sparse_kv_attn_func(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *, scale=None,
                        dispatch_to_custom_ops=True):
    """Attention that drops the keys a boolean key-padding mask marks False
    (src/para_attn/sparse_attn.py:14-69). Both dispatch settings run the same kernel."""
    return para_attn_ops.attention_forward_sparse_kv(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p,
                                                     is_causal=is_causal, scale=scale)


class SparseKVAttnMode(BaseTorchFunctionMode):
    """Routes ``F.scaled_dot_product_attention`` to ``sparse_kv_attn_func``
    (src/para_attn/sparse_attn.py:607-640)."""

    disabled = False

    @torch.compiler.disable
    def __init__(self, *, dispatch_to_custom_ops=True):
        super().__init__()
        self._dispatch_to_custom_ops = dispatch_to_custom_ops

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = {} if kwargs is None else kwargs
        if SparseKVAttnMode.disabled:
            return base_handle_torch_function(func, types, args, kwargs)
        if func is F.scaled_dot_product_attention:
            return sparse_kv_attn_func(*args, **kwargs, dispatch_to_custom_ops=self._dispatch_to_custom_ops)
        return base_handle_torch_function(func, types, args, kwargs)

    @classmethod
    @contextlib.contextmanager
    def disable(cls):
        old_disabled = cls._set_disabled(True)
        try:
            yield
        finally:
            cls._set_disabled(old_disabled)

    @classmethod
    @torch.compiler.disable
    def _set_disabled(cls, value):
        old_disabled = cls.disabled
        cls.disabled = value
        return old_disabled


class InBatchAttnMode(_AttnModeBase):
    disabled = False

    @torch.compiler.disable
    def __init__(self):
        super().__init__()
        self._skip_small_kv = False

    def _call_attn_func(self, *args, **kwargs):
        return in_batch_attn_func(*args, **kwargs)
