"""First Block Cache: state, decision and cached block runner with the reference's names
(src/para_attn/first_block_cache/utils.py:12-451).

The bookkeeping (``CacheContext``, step counting, alternate cache, warm-up, SLG) is host-only
Python like the reference's. What touches the device is different: forming the first-block
residual, the two mean-absolute reductions of ``are_two_tensors_similar`` and storing the
residual for the next step are ONE launch of ``pa_fbc_residual_diff`` (the reference issues
about eight elementwise/reduction kernels for the same result), and applying / forming the
cached residual is ``pa_fbc_axpy``. Rounding points follow the reference's bf16 arithmetic so
that the skip/compute decision is the same at every step.
"""
from __future__ import annotations

import contextlib
import dataclasses
from collections import defaultdict
from typing import Any, DefaultDict, Dict, List, Optional, Union

import torch

from .. import _lib as L
from .. import primitives as DP
from .taylorseer import TaylorSeer

_DTYPES = {torch.bfloat16: L.PA_BF16, torch.float16: L.PA_F16}


@dataclasses.dataclass
class CacheContext:
    residual_diff_threshold: Union[torch.Tensor, float] = 0.0
    alter_residual_diff_threshold: Optional[Union[torch.Tensor, float]] = None

    downsample_factor: int = 1

    enable_alter_cache: bool = False
    num_inference_steps: int = -1
    warmup_steps: int = 0

    enable_taylorseer: bool = False
    taylorseer_kwargs: Dict[str, Any] = dataclasses.field(default_factory=dict)

    slg_layers: Optional[List[int]] = None
    slg_start: float = 0.0
    slg_end: float = 0.1

    buffers: Dict[str, Any] = dataclasses.field(default_factory=dict)
    incremental_name_counters: DefaultDict[str, int] = dataclasses.field(default_factory=lambda: defaultdict(int))

    executed_steps: int = 0
    is_alter_cache: bool = True

    taylorseer: Optional[TaylorSeer] = None
    alter_taylorseer: Optional[TaylorSeer] = None

    def __post_init__(self):
        if self.enable_taylorseer:
            self.taylorseer = TaylorSeer(**self.taylorseer_kwargs)
            if self.enable_alter_cache:
                self.alter_taylorseer = TaylorSeer(**self.taylorseer_kwargs)

    def get_incremental_name(self, name=None):
        if name is None:
            name = "default"
        idx = self.incremental_name_counters[name]
        self.incremental_name_counters[name] += 1
        return f"{name}_{idx}"

    def reset_incremental_names(self):
        self.incremental_name_counters.clear()

    def get_residual_diff_threshold(self):
        if self.enable_alter_cache and self.is_alter_cache and self.alter_residual_diff_threshold is not None:
            residual_diff_threshold = self.alter_residual_diff_threshold
        else:
            residual_diff_threshold = self.residual_diff_threshold
        if isinstance(residual_diff_threshold, torch.Tensor):
            residual_diff_threshold = residual_diff_threshold.item()
        return residual_diff_threshold

    def _name(self, name):
        if self.enable_alter_cache and self.is_alter_cache:
            return f"{name}_alter"
        return name

    def get_buffer(self, name):
        return self.buffers.get(self._name(name))

    def set_buffer(self, name, buffer):
        self.buffers[self._name(name)] = buffer

    def remove_buffer(self, name):
        self.buffers.pop(self._name(name), None)

    def clear_buffers(self):
        self.buffers.clear()

    def mark_step_begin(self):
        if not self.enable_alter_cache:
            self.executed_steps += 1
        else:
            self.is_alter_cache = not self.is_alter_cache
            if not self.is_alter_cache:
                self.executed_steps += 1
        if self.enable_taylorseer:
            self.get_taylorseer().mark_step_begin()

    def get_taylorseer(self):
        if self.enable_alter_cache and self.is_alter_cache:
            return self.alter_taylorseer
        return self.taylorseer

    def is_slg_enabled(self):
        return self.slg_layers is not None

    def slg_should_skip_block(self, block_idx):
        if not self.enable_alter_cache or not self.is_alter_cache:
            return False
        if self.slg_layers is None:
            return False
        if self.slg_start <= 0.0 and self.slg_end >= 1.0:
            return False
        num_inference_steps = self.num_inference_steps
        assert num_inference_steps >= 0, "num_inference_steps must be non-negative"
        return (
            block_idx in self.slg_layers
            and num_inference_steps * self.slg_start <= self.get_current_step() < num_inference_steps * self.slg_end
        )

    def get_current_step(self):
        return self.executed_steps - 1

    def is_in_warmup(self):
        return self.get_current_step() < self.warmup_steps


_current_cache_context = None


def create_cache_context(*args, **kwargs):
    return CacheContext(*args, **kwargs)


def get_current_cache_context():
    return _current_cache_context


def set_current_cache_context(cache_context=None):
    global _current_cache_context
    _current_cache_context = cache_context


@contextlib.contextmanager
def cache_context(cache_context):
    global _current_cache_context
    old_cache_context = _current_cache_context
    _current_cache_context = cache_context
    try:
        yield
    finally:
        _current_cache_context = old_cache_context


def _ctx() -> CacheContext:
    cache_context = get_current_cache_context()
    assert cache_context is not None, "cache_context must be set before"
    return cache_context


def get_residual_diff_threshold():
    return _ctx().get_residual_diff_threshold()


def get_buffer(name):
    return _ctx().get_buffer(name)


def set_buffer(name, buffer):
    _ctx().set_buffer(name, buffer)


def remove_buffer(name):
    _ctx().remove_buffer(name)


def mark_step_begin():
    _ctx().mark_step_begin()


def is_taylorseer_enabled():
    return _ctx().enable_taylorseer


def get_taylorseer():
    return _ctx().get_taylorseer()


def is_slg_enabled():
    return _ctx().is_slg_enabled()


def slg_should_skip_block(block_idx):
    return _ctx().slg_should_skip_block(block_idx)


def is_in_warmup():
    return _ctx().is_in_warmup()


def get_downsample_factor():
    return _ctx().downsample_factor


# --------------------------------------------------------------------------------------------
# device work
# --------------------------------------------------------------------------------------------
_scratch: Dict[int, torch.Tensor] = {}


def _scratch_for(device: torch.device) -> torch.Tensor:
    buf = _scratch.get(device.index)
    if buf is None:
        buf = torch.zeros(int(L.load().pa_fbc_scratch_bytes()), dtype=torch.uint8, device=device)
        _scratch[device.index] = buf
    return buf


def _kernel_ok(*tensors) -> bool:
    t0 = tensors[0]
    return all(
        t is None or (t.device.type == "cuda" and t.dtype in _DTYPES and t.dtype == t0.dtype and t.is_contiguous())
        for t in tensors
    )


def _require_cuda(t: torch.Tensor):
    if t.device.type != "cuda":
        raise RuntimeError("First Block Cache kernels need CUDA tensors; there is no CPU path in this package")


def fused_residual_diff(h1: torch.Tensor, h0: torch.Tensor, prev: Optional[torch.Tensor], *, downsample: int = 1,
                        store: bool = True):
    """One launch: ``cur = h1 - h0`` (rounded to the tensors' dtype, optionally only every
    ``downsample``-th channel), and if ``prev`` is given the fp32 sums / rounded means / rounded
    ratio of ``are_two_tensors_similar(prev, cur)`` (src/para_attn/first_block_cache/utils.py:228-233).

    Returns ``(cur or None, result)`` with ``result`` a 5-float device tensor
    [sum|prev-cur|, sum|prev|, mean_diff, mean_prev, mean_diff/mean_prev]."""
    _require_cuda(h1)
    assert h1.shape == h0.shape and h1.dtype == h0.dtype
    if not _kernel_ok(h1, h0, prev):
        raise NotImplementedError("fused_residual_diff needs contiguous CUDA bf16/f16 tensors of one dtype")
    cols = h1.shape[-1]
    rows = h1.numel() // cols
    cols_ds = (cols + downsample - 1) // downsample
    new_shape = tuple(h1.shape[:-1]) + (cols_ds,)
    if prev is not None:
        assert tuple(prev.shape) == new_shape
    cur = torch.empty(new_shape, dtype=h1.dtype, device=h1.device) if store else None
    result = torch.empty(5, dtype=torch.float32, device=h1.device)
    L.check(L.load().pa_fbc_residual_diff(
        h1.data_ptr(), h0.data_ptr(), prev.data_ptr() if prev is not None else None,
        cur.data_ptr() if cur is not None else None, rows, cols, downsample, _DTYPES[h1.dtype], result.data_ptr(),
        _scratch_for(h1.device).data_ptr(), torch.cuda.current_stream(h1.device).cuda_stream))
    return cur, result


def _axpy(a: torch.Tensor, b: torch.Tensor, sub: bool) -> torch.Tensor:
    _require_cuda(a)
    if _kernel_ok(a, b) and a.shape == b.shape and a.numel() % 8 == 0 and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0:
        out = torch.empty_like(a)
        L.check(L.load().pa_fbc_axpy(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), 1 if sub else 0,
                                     _DTYPES[a.dtype], torch.cuda.current_stream(a.device).cuda_stream))
        return out
    # shapes the vector kernel does not take (odd sizes, fp32, broadcasting): same arithmetic in ATen
    return (a - b if sub else a + b).contiguous()


def _decide(result: torch.Tensor, dtype: torch.dtype, threshold: float, parallelized: bool) -> bool:
    if parallelized:
        # the reference averages each rounded mean over the default group (utils.py:230-232)
        means = result[2:4].to(dtype)
        means = DP.all_reduce_sync(means, "avg")
        diff = means[0] / means[1]
    else:
        diff = result[4]
    return diff.item() < threshold


def are_two_tensors_similar(t1, t2, *, threshold, parallelized=False):
    """mean|t1 - t2| / mean|t1| < threshold with the reference's rounding (utils.py:220-234)."""
    if threshold <= 0.0:
        return False
    if t1.shape != t2.shape:
        return False
    _require_cuda(t1)
    zero = torch.zeros_like(t2)
    _, result = fused_residual_diff(t2.contiguous(), zero, t1.contiguous(), store=False)
    return _decide(result, t1.dtype, threshold, parallelized)


def apply_prev_hidden_states_residual(hidden_states, encoder_hidden_states=None):
    if is_taylorseer_enabled():
        # extrapolated residual + hidden states in one launch; the encoder states pass through
        # unchanged (src/para_attn/first_block_cache/utils.py:238-243)
        return get_taylorseer().approximate_value(add=hidden_states.contiguous()), encoder_hidden_states
    hidden_states_residual = get_hidden_states_residual()
    assert hidden_states_residual is not None, "hidden_states_residual must be set before"
    hidden_states = _axpy(hidden_states_residual, hidden_states.contiguous(), sub=False)

    if encoder_hidden_states is not None:
        encoder_hidden_states_residual = get_encoder_hidden_states_residual()
        assert encoder_hidden_states_residual is not None, "encoder_hidden_states_residual must be set before"
        encoder_hidden_states = _axpy(encoder_hidden_states_residual, encoder_hidden_states.contiguous(), sub=False)

    return hidden_states, encoder_hidden_states


def get_can_use_cache(first_hidden_states_residual, parallelized=False):
    """Reference-shaped entry (utils.py:269-286) for callers that already hold the residual."""
    if is_in_warmup():
        return False
    threshold = get_residual_diff_threshold()
    if threshold <= 0.0:
        return False
    downsample_factor = get_downsample_factor()
    if downsample_factor > 1:
        first_hidden_states_residual = first_hidden_states_residual[..., ::downsample_factor]
    prev_first_hidden_states_residual = get_first_hidden_states_residual()
    can_use_cache = prev_first_hidden_states_residual is not None and are_two_tensors_similar(
        prev_first_hidden_states_residual,
        first_hidden_states_residual,
        threshold=threshold,
        parallelized=parallelized,
    )
    return can_use_cache


def set_first_hidden_states_residual(first_hidden_states_residual):
    downsample_factor = get_downsample_factor()
    if downsample_factor > 1:
        first_hidden_states_residual = first_hidden_states_residual[..., ::downsample_factor]
        first_hidden_states_residual = first_hidden_states_residual.contiguous()
    set_buffer("first_hidden_states_residual", first_hidden_states_residual)


def get_first_hidden_states_residual():
    return get_buffer("first_hidden_states_residual")


def set_hidden_states_residual(hidden_states_residual):
    if is_taylorseer_enabled():
        get_taylorseer().update(hidden_states_residual)
    else:
        set_buffer("hidden_states_residual", hidden_states_residual)


def get_hidden_states_residual():
    if is_taylorseer_enabled():
        return get_taylorseer().approximate_value()
    return get_buffer("hidden_states_residual")


def set_encoder_hidden_states_residual(encoder_hidden_states_residual):
    if is_taylorseer_enabled():
        return
    set_buffer("encoder_hidden_states_residual", encoder_hidden_states_residual)


def get_encoder_hidden_states_residual():
    return get_buffer("encoder_hidden_states_residual")


def first_block_decision(hidden_states, original_hidden_states, parallelized=False) -> bool:
    """Fused form of utils.py:359-381: residual of the first block, comparison with the previous
    step's, and - on a miss - storing it as the new reference. Returns can_use_cache."""
    ds = get_downsample_factor()
    h1 = hidden_states.contiguous()
    h0 = original_hidden_states.contiguous()
    threshold = get_residual_diff_threshold()
    prev = get_first_hidden_states_residual()
    compare = (not is_in_warmup()) and threshold > 0.0 and prev is not None
    if compare:
        cols_ds = (h1.shape[-1] + ds - 1) // ds
        compare = tuple(prev.shape) == tuple(h1.shape[:-1]) + (cols_ds,)
    cur, result = fused_residual_diff(h1, h0, prev if compare else None, downsample=ds, store=True)
    can_use_cache = compare and _decide(result, h1.dtype, threshold, parallelized)
    if not can_use_cache:
        set_buffer("first_hidden_states_residual", cur)
    return can_use_cache


class CachedTransformerBlocks(torch.nn.Module):
    def __init__(
        self,
        transformer_blocks,
        single_transformer_blocks=None,
        *,
        transformer=None,
        return_hidden_states_first=True,
        return_hidden_states_only=False,
    ):
        super().__init__()

        self.transformer = transformer
        self.transformer_blocks = transformer_blocks
        self.single_transformer_blocks = single_transformer_blocks
        self.return_hidden_states_first = return_hidden_states_first
        self.return_hidden_states_only = return_hidden_states_only

    def _unpack(self, hidden_states, encoder_hidden_states):
        if not isinstance(hidden_states, torch.Tensor):
            hidden_states, encoder_hidden_states = hidden_states
            if not self.return_hidden_states_first:
                hidden_states, encoder_hidden_states = encoder_hidden_states, hidden_states
        return hidden_states, encoder_hidden_states

    def forward(self, hidden_states, encoder_hidden_states, *args, **kwargs):
        original_hidden_states = hidden_states
        first_transformer_block = self.transformer_blocks[0]
        hidden_states = first_transformer_block(hidden_states, encoder_hidden_states, *args, **kwargs)
        hidden_states, encoder_hidden_states = self._unpack(hidden_states, encoder_hidden_states)

        mark_step_begin()
        can_use_cache = first_block_decision(
            hidden_states,
            original_hidden_states,
            parallelized=self.transformer is not None and getattr(self.transformer, "_is_parallelized", False),
        )
        del original_hidden_states

        if can_use_cache:
            hidden_states, encoder_hidden_states = apply_prev_hidden_states_residual(
                hidden_states, encoder_hidden_states
            )
        else:
            (
                hidden_states,
                encoder_hidden_states,
                hidden_states_residual,
                encoder_hidden_states_residual,
            ) = self.call_remaining_transformer_blocks(hidden_states, encoder_hidden_states, *args, **kwargs)
            set_hidden_states_residual(hidden_states_residual)
            set_encoder_hidden_states_residual(encoder_hidden_states_residual)

        return (
            hidden_states
            if self.return_hidden_states_only
            else (
                (hidden_states, encoder_hidden_states)
                if self.return_hidden_states_first
                else (encoder_hidden_states, hidden_states)
            )
        )

    def call_remaining_transformer_blocks(self, hidden_states, encoder_hidden_states, *args, **kwargs):
        original_hidden_states = hidden_states
        original_encoder_hidden_states = encoder_hidden_states
        slg = is_slg_enabled()
        for i, block in enumerate(self.transformer_blocks[1:]):
            if slg and slg_should_skip_block(i + 1):
                continue
            hidden_states = block(hidden_states, encoder_hidden_states, *args, **kwargs)
            hidden_states, encoder_hidden_states = self._unpack(hidden_states, encoder_hidden_states)
        if self.single_transformer_blocks is not None:
            hidden_states = torch.cat([encoder_hidden_states, hidden_states], dim=1)
            for i, block in enumerate(self.single_transformer_blocks):
                if slg and slg_should_skip_block(len(self.transformer_blocks) + i):
                    continue
                hidden_states = block(hidden_states, *args, **kwargs)
            encoder_hidden_states, hidden_states = hidden_states.split(
                [encoder_hidden_states.shape[1], hidden_states.shape[1] - encoder_hidden_states.shape[1]], dim=1
            )

        hidden_states = hidden_states.reshape(-1).contiguous().reshape(original_hidden_states.shape)
        hidden_states_residual = _axpy(hidden_states, original_hidden_states.contiguous(), sub=True)
        encoder_hidden_states_residual = None
        if encoder_hidden_states is not None:
            encoder_hidden_states = (
                encoder_hidden_states.reshape(-1).contiguous().reshape(original_encoder_hidden_states.shape)
            )
            encoder_hidden_states_residual = _axpy(
                encoder_hidden_states, original_encoder_hidden_states.contiguous(), sub=True)

        return hidden_states, encoder_hidden_states, hidden_states_residual, encoder_hidden_states_residual
