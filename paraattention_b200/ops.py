"""Attention custom ops, same names and signatures as the reference's ``para_attn.ops``
(src/para_attn/ops/__init__.py:160-245), backed by the sm_100a kernels of libpa_b200.

``torch.ops.para_attn.attention_forward_with_lse(q, k, v, attn_mask=None, dropout_p=0.0,
is_causal=False, *, scale=None) -> (out, lse)`` and ``attention_forward(...) -> out``.
Where the reference picks one of PyTorch's flash / efficient / cuDNN SDPA backends
(:112-157), these ops launch one tcgen05 flash-attention kernel. They are CUDA-only: a CPU
tensor raises, nothing falls back to PyTorch math.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from . import _lib as L
from . import _status
from . import config

__all__ = [
    "attention_forward_with_lse",
    "attention_forward",
    "attention_forward_sparse_kv",
    "cp_attention_forward",
    "key_mask_of",
    "pack_key_mask",
    "merge_out_lse_",
    "raw_attention_forward",
    "qkv_prepare",
]

_DTYPES = {torch.bfloat16: L.PA_BF16, torch.float16: L.PA_F16}


def _check_inputs(query, key, value, attn_mask, dropout_p, is_causal):
    assert query.device.type == "cuda", "Must be CUDA tensors"  # as src/para_attn/ops/__init__.py:123
    assert query.ndim == 4 and key.ndim == 4 and value.ndim == 4, "query, key and value must be [B, H, S, D]"
    if query.dtype not in _DTYPES or key.dtype != query.dtype or value.dtype != query.dtype:
        raise NotImplementedError(f"attention dtype {query.dtype}: only bfloat16 and float16 are built")
    if attn_mask is not None:
        raise NotImplementedError("attn_mask: only boolean key-padding masks are built into the sm_100a attention "
                                  "kernel (torch.ops.para_attn.attention_forward_sparse_kv)")
    if dropout_p != 0.0:
        raise NotImplementedError("dropout_p must be 0: the library is forward/inference only")
    D = query.shape[-1]
    if D not in (64, 128) or key.shape[-1] != D or value.shape[-1] != D:
        raise NotImplementedError(f"head_dim {D}: only 64 and 128 are built (query, key and value alike)")
    assert key.shape[:2] == query.shape[:2] and value.shape == key.shape, "mismatched batch/head/key shapes"


def _tma_ready(x: torch.Tensor) -> torch.Tensor:
    """Return x itself if the kernel can address it in place (unit stride on head_dim, 16-byte
    aligned base and strides, no broadcast dims), else a contiguous copy."""
    ok = x.stride(-1) == 1 and x.data_ptr() % 16 == 0
    for i in range(3):
        s = x.stride(i)
        ok = ok and (x.shape[i] == 1 or (s > 0 and (s * x.element_size()) % 16 == 0))
    return x if ok else x.contiguous()


def key_mask_of(attn_mask: Optional[torch.Tensor], batch: int, keys: int) -> Optional[torch.Tensor]:
    """The [batch, keys] boolean key-padding mask that ``attn_mask`` stands for, or None if it is
    not one. The reference's sparse-KV path reads one row of key flags per batch element
    (``while m.ndim > 1: m = m[0]``, src/para_attn/ops/__init__.py:279-280); here the mask must
    say so itself: boolean, broadcastable to [batch, 1, 1, keys] with size-1 head and query dims."""
    if attn_mask is None or attn_mask.dtype != torch.bool or attn_mask.ndim > 4 or attn_mask.ndim < 1:
        return None
    m = attn_mask
    while m.ndim < 4:
        m = m.unsqueeze(0)
    if m.shape[1] != 1 or m.shape[2] != 1 or m.shape[3] != keys or m.shape[0] not in (1, batch):
        return None
    return m[:, 0, 0, :].expand(batch, keys)


# Packed words of the last few masks. A diffusion transformer hands the same mask tensor to every
# attention of a forward (60 calls for a HunyuanVideo-shaped model): it is packed once. An entry
# keeps its mask tensor alive, so "same storage address, same version counter, same layout" can
# only mean the same contents.
_PACK_CACHE: list = []
_PACK_CACHE_SIZE = 4


def pack_key_mask(key_mask: torch.Tensor, n_chunks: int, rows: int) -> torch.Tensor:
    """pa_pack_key_mask: [batch, n_chunks * rows] bool -> [batch, n_chunks, ceil(rows / 64)] words
    (int64 storage) as the attention entry points read them."""
    assert key_mask.dtype == torch.bool and key_mask.ndim == 2 and key_mask.shape[1] == n_chunks * rows
    assert key_mask.device.type == "cuda", "Must be CUDA tensors"
    ident = (key_mask.data_ptr(), key_mask._version, tuple(key_mask.shape), key_mask.stride(), n_chunks, rows,
             key_mask.device.index)
    for i, (k, _, words) in enumerate(_PACK_CACHE):
        if k == ident:
            if i:
                _PACK_CACHE.insert(0, _PACK_CACHE.pop(i))
            return words
    m = key_mask.contiguous()
    out = torch.empty((m.shape[0], n_chunks, (rows + 63) // 64), dtype=torch.int64, device=m.device)
    L.check(L.load().pa_pack_key_mask(m.data_ptr(), m.stride(0), m.shape[0], n_chunks, rows, out.data_ptr(),
                                      torch.cuda.current_stream(m.device).cuda_stream))
    _PACK_CACHE.insert(0, (ident, key_mask, out))
    del _PACK_CACHE[_PACK_CACHE_SIZE:]
    return out


_SPLIT_WS: dict = {}


def split_workspace(device: torch.device, stream: int) -> torch.Tensor:
    """Scratch memory for launches that split their last wave (pa_attn_args.workspace), one
    buffer per device and stream: launches that may overlap must not share it."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _SPLIT_WS.get(key)
    if ws is None:
        if len(_SPLIT_WS) >= 16:  # (streams come and go)
            _SPLIT_WS.clear()
        ws = torch.empty(int(L.load().pa_attn_workspace_bytes()), dtype=torch.uint8, device=device)
        _SPLIT_WS[key] = ws
    return ws


def raw_attention_forward(query, key, value, scale: Optional[float], need_lse: bool,
                          status: Optional[torch.Tensor] = None, is_causal: bool = False,
                          key_mask: Optional[torch.Tensor] = None):
    """Launch pa_attn_fwd on the current stream. Output memory is [B, S, H, D] viewed as
    [B, H, S, D], the layout PyTorch's flash backend returns, so that the usual
    ``transpose(1, 2).flatten(2)`` that follows attention is free."""
    B, H, Sq, D = query.shape
    Skv = key.shape[2]
    q, k, v = _tma_ready(query), _tma_ready(key), _tma_ready(value)
    out = torch.empty((B, Sq, H, D), dtype=query.dtype, device=query.device).transpose(1, 2)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=query.device) if need_lse else None
    a = L.AttnArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.batch, a.heads, a.seq_q, a.seq_kv, a.head_dim = B, H, Sq, Skv, D
    a.dtype = _DTYPES[query.dtype]
    a.is_causal = 1 if is_causal else 0
    a.scale = (1.0 / math.sqrt(D)) if scale is None else float(scale)
    for i in range(3):
        a.q_stride[i], a.k_stride[i], a.v_stride[i], a.o_stride[i] = q.stride(i), k.stride(i), v.stride(i), out.stride(i)
    # Without a status word of the caller's, the process-wide one of this device: a wait that ran
    # out in an earlier launch is raised here, and this launch's outcome is queued for the next.
    mirror = None
    if status is None:
        mirror = _status.single_gpu_status(query.device)
        mirror.check()
        status = mirror.word
    a.status = status.data_ptr()
    a.wait_limit_ns = 0
    bits = pack_key_mask(key_mask, 1, Skv) if key_mask is not None else None
    a.key_bits = bits.data_ptr() if bits is not None else None
    stream = torch.cuda.current_stream(query.device).cuda_stream
    if config.attention.split_last_wave and not is_causal:
        ws = split_workspace(query.device, stream)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    L.check(L.load().pa_attn_fwd(C.byref(a), stream))
    if mirror is not None:
        mirror.refresh()
    return out, lse


@torch.library.custom_op("para_attn::attention_forward_with_lse", mutates_args=(), device_types=("cuda",))
def attention_forward_with_lse(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_mask: Optional[torch.Tensor] = None,
    dropout_p: float = 0.0,
    is_causal: bool = False,
    *,
    scale: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    _check_inputs(query, key, value, attn_mask, dropout_p, is_causal)
    out, lse = raw_attention_forward(query, key, value, scale, True, is_causal=is_causal)
    return out, lse


@torch.library.register_fake("para_attn::attention_forward_with_lse")
def _(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *, scale=None):
    B, H, Sq, D = query.shape
    out = query.new_empty((B, Sq, H, D)).transpose(1, 2)
    lse = query.new_empty((B, H, Sq), dtype=torch.float32)
    return out, lse


@torch.library.custom_op("para_attn::attention_forward", mutates_args=(), device_types=("cuda",))
def attention_forward(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_mask: Optional[torch.Tensor] = None,
    dropout_p: float = 0.0,
    is_causal: bool = False,
    *,
    scale: Optional[float] = None,
) -> torch.Tensor:
    _check_inputs(query, key, value, attn_mask, dropout_p, is_causal)
    out, _ = raw_attention_forward(query, key, value, scale, False, is_causal=is_causal)
    return out


@torch.library.register_fake("para_attn::attention_forward")
def _(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *, scale=None):
    B, H, Sq, D = query.shape
    return query.new_empty((B, Sq, H, D)).transpose(1, 2)


@torch.library.custom_op("para_attn::attention_forward_sparse_kv", mutates_args=(), device_types=("cuda",))
def attention_forward_sparse_kv(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_mask: Optional[torch.Tensor] = None,
    dropout_p: float = 0.0,
    is_causal: bool = False,
    *,
    scale: Optional[float] = None,
) -> torch.Tensor:
    """Attention over the keys a boolean key-padding mask keeps
    (src/para_attn/ops/__init__.py:248-343). The reference gathers the kept keys per batch element
    and runs SDPA on each; here the kernel masks the dropped keys in place, one launch for the
    whole batch. A query whose keys are all dropped yields zeros."""
    if attn_mask is None:
        _check_inputs(query, key, value, None, dropout_p, is_causal)
        return raw_attention_forward(query, key, value, scale, False, is_causal=is_causal)[0]
    assert attn_mask.dtype == torch.bool, "attn_mask must be a boolean tensor"
    assert not is_causal, "is_causal is not supported with sparse kv"
    _check_inputs(query, key, value, None, dropout_p, is_causal)
    km = key_mask_of(attn_mask, query.shape[0], key.shape[2])
    if km is None:
        raise NotImplementedError(
            f"attn_mask of shape {tuple(attn_mask.shape)}: expected a key-padding mask broadcastable to "
            f"[{query.shape[0]}, 1, 1, {key.shape[2]}]")
    return raw_attention_forward(query, key, value, scale, False, key_mask=km)[0]


@torch.library.register_fake("para_attn::attention_forward_sparse_kv")
def _(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, *, scale=None):
    B, H, Sq, D = query.shape
    return query.new_empty((B, Sq, H, D)).transpose(1, 2)


# (the expected values of the exchange counters advance on the host with every call, so a
# replayed CUDA graph of this op would wait for counts that never come: tagged accordingly)
@torch.library.custom_op("para_attn::cp_attention_forward", mutates_args=(), device_types=("cuda",),
                         tags=(torch.Tag.cudagraph_unsafe,))
def cp_attention_forward(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    key_mask: Optional[torch.Tensor],
    is_causal: bool,
    scale: Optional[float],
    engine_id: int,
) -> torch.Tensor:
    """One context-parallel attention call of this rank (exchange + chunked attention + output
    scatter) as a custom op, so that the Ring / Ulysses / Unified modes stay traceable: the
    engine (process group, mesh position, workspace) is named by an integer
    (``_cp_engine.engine_id``). No counterpart in the reference, whose collectives are traceable
    functional collectives (src/para_attn/primitives.py:72-78)."""
    from . import _cp_engine

    return _cp_engine.engine_by_id(engine_id).attention(query, key, value, scale, is_causal=is_causal,
                                                         key_mask=key_mask)


@torch.library.register_fake("para_attn::cp_attention_forward")
def _(query, key, value, key_mask, is_causal, scale, engine_id):
    B, H, Sq, D = query.shape
    return query.new_empty((B, Sq, H, D)).transpose(1, 2)


def qkv_prepare(q: torch.Tensor, k: torch.Tensor, v: Optional[torch.Tensor], q_weight: Optional[torch.Tensor] = None,
                k_weight: Optional[torch.Tensor] = None, rotary: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, *,
                eps: float = 1e-6, out: Optional[Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]] = None,
                row_offset: int = 0):
    """What a transformer block does to q, k, v between their projections and attention, in one
    launch of pa_qkv_prep: per-head RMSNorm of q and k (``x * rsqrt(mean(x^2) + eps)`` rounded to
    the dtype, times the per-channel weight), rotary embedding of both (``rotary = (cos, sin)``,
    fp32 [rows of the whole sequence, D]; adjacent elements are the rotation pairs), and placement
    into [B, H, S, D] views of [B, S, H, D] buffers - the layout the attention ops like best.

    q, k, v: [B, H, S, D] views with contiguous D (projection outputs viewed per head). With
    ``out = (q_buf, k_buf, v_buf)`` ([B, H, S_total, D] views, S_total >= row_offset + S) the rows
    [row_offset, row_offset + S) of those buffers are written and the rotary tables are read
    from row ``row_offset`` on, which is how the streams of a joint-attention block land in one
    buffer without a concatenation. Returns the three destination views (the written rows)."""
    assert q.device.type == "cuda", "Must be CUDA tensors"
    assert q.ndim == 4 and k.shape == q.shape and (v is None or v.shape == q.shape), "q, k, v must be [B, H, S, D] alike"
    if q.dtype not in _DTYPES or k.dtype != q.dtype or (v is not None and v.dtype != q.dtype):
        raise NotImplementedError(f"qkv_prepare dtype {q.dtype}: only bfloat16 and float16 are built")
    B, H, S, D = q.shape
    if D not in (64, 128):
        raise NotImplementedError(f"head_dim {D}: only 64 and 128 are built")
    ins = [q, k, v]
    for i, t in enumerate(ins):
        if t is not None and t.stride(-1) != 1:
            ins[i] = t.contiguous()
    if out is None:
        out = tuple(torch.empty((B, S, H, D), dtype=q.dtype, device=q.device).transpose(1, 2) if t is not None else None
                    for t in ins)
        row_offset_out = 0
    else:
        row_offset_out = row_offset
        for t, o in zip(ins, out):
            assert (t is None) == (o is None)
            assert o is None or (o.ndim == 4 and o.shape[0] == B and o.shape[1] == H and o.shape[3] == D and
                                 o.shape[2] >= row_offset + S and o.stride(-1) == 1 and o.dtype == q.dtype)
    a = L.QkvPrepArgs()
    dsts = []
    for name, t, o in zip("qkv", ins, out):
        if t is None:
            dsts.append(None)
            continue
        dst = o[:, :, row_offset_out:row_offset_out + S]
        dsts.append(dst)
        setattr(a, name, t.data_ptr())
        setattr(a, name + "_out", dst.data_ptr())
        for j, dim in enumerate((0, 2, 1)):  # (batch, row, head)
            getattr(a, name + "_stride")[j] = t.stride(dim)
            getattr(a, name + "_out_stride")[j] = dst.stride(dim)
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            assert w.shape == (D,) and w.dtype == q.dtype and w.is_contiguous() and w.device == q.device
            setattr(a, name, w.data_ptr())
    if rotary is not None:
        cos, sin = rotary
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
        assert cos.shape == sin.shape and cos.ndim == 2 and cos.shape[1] == D and cos.shape[0] >= row_offset + S
        a.cos, a.sin = cos.data_ptr(), sin.data_ptr()
    a.table_row0 = row_offset
    a.batch, a.rows, a.heads, a.head_dim = B, S, H, D
    a.dtype = _DTYPES[q.dtype]
    a.eps = eps
    L.check(L.load().pa_qkv_prep(C.byref(a), torch.cuda.current_stream(q.device).cuda_stream))
    return tuple(dsts)


def merge_out_lse_(acc_out: torch.Tensor, acc_lse: torch.Tensor, block_out: torch.Tensor,
                   block_lse: torch.Tensor) -> None:
    """In-place ``_SDPAMerger._merge_one`` (torch/distributed/tensor/experimental/
    _context_parallel/_attention.py:182-183): acc_out fp32 [..., S, D], acc_lse fp32 [..., S]."""
    assert acc_out.dtype == torch.float32 and acc_lse.dtype == torch.float32 and block_lse.dtype == torch.float32
    assert acc_out.is_contiguous() and acc_lse.is_contiguous() and block_out.is_contiguous() and block_lse.is_contiguous()
    assert acc_out.shape == block_out.shape and acc_lse.shape == block_lse.shape == acc_out.shape[:-1]
    code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[block_out.dtype]
    L.check(L.load().pa_merge_out_lse(acc_out.data_ptr(), acc_lse.data_ptr(), block_out.data_ptr(), block_lse.data_ptr(),
                                      acc_lse.numel(), acc_out.shape[-1], code,
                                      torch.cuda.current_stream(acc_out.device).cuda_stream))
