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
    """State of one cached denoising run. The constructor arguments are the reference's
    (utils.py:12-36); ``apply_cache_on_pipe(**kwargs)`` forwards to them."""

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
        if not self.enable_taylorseer:
            return
        # one extrapolator per cache: the alternate cache (second forward of a step) has its own
        self.taylorseer = TaylorSeer(**self.taylorseer_kwargs)
        self.alter_taylorseer = TaylorSeer(**self.taylorseer_kwargs) if self.enable_alter_cache else None

    # -- which of the two caches is current --------------------------------------------------
    @property
    def _on_alter(self) -> bool:
        return self.enable_alter_cache and self.is_alter_cache

    def _name(self, name: str) -> str:
        return name + "_alter" if self._on_alter else name

    def get_taylorseer(self):
        return self.alter_taylorseer if self._on_alter else self.taylorseer

    def get_residual_diff_threshold(self):
        use_alter = self._on_alter and self.alter_residual_diff_threshold is not None
        threshold = self.alter_residual_diff_threshold if use_alter else self.residual_diff_threshold
        return threshold.item() if isinstance(threshold, torch.Tensor) else threshold

    # -- named buffers --------------------------------------------------------------------------
    def get_incremental_name(self, name=None):
        key = "default" if name is None else name
        index = self.incremental_name_counters[key]
        self.incremental_name_counters[key] = index + 1
        return f"{key}_{index}"

    def reset_incremental_names(self):
        self.incremental_name_counters.clear()

    def get_buffer(self, name):
        return self.buffers.get(self._name(name))

    def set_buffer(self, name, buffer):
        self.buffers[self._name(name)] = buffer

    def remove_buffer(self, name):
        self.buffers.pop(self._name(name), None)

    def clear_buffers(self):
        self.buffers.clear()

    # -- steps ------------------------------------------------------------------------------------
    def mark_step_begin(self):
        """Called once per transformer forward. With the alternate cache the two forwards of a
        step take turns (the flag starts True, so the first forward lands on the main cache)
        and only the main one counts a step (utils.py:83-92)."""
        if self.enable_alter_cache:
            self.is_alter_cache = not self.is_alter_cache
        if not self._on_alter:
            self.executed_steps += 1
        if self.enable_taylorseer:
            self.get_taylorseer().mark_step_begin()

    def get_current_step(self):
        return self.executed_steps - 1

    def is_in_warmup(self):
        return self.get_current_step() < self.warmup_steps

    # -- skip-layer guidance ----------------------------------------------------------------------
    def is_slg_enabled(self):
        return self.slg_layers is not None

    def slg_should_skip_block(self, block_idx):
        """Blocks listed in ``slg_layers`` are left out on the alternate forward while the step is
        inside [slg_start, slg_end) of the schedule (utils.py:102-116)."""
        if not self._on_alter or self.slg_layers is None:
            return False
        if self.slg_start <= 0.0 and self.slg_end >= 1.0:
            return False
        total = self.num_inference_steps
        assert total >= 0, "num_inference_steps must be non-negative"
        in_window = total * self.slg_start <= self.get_current_step() < total * self.slg_end
        return in_window and block_idx in self.slg_layers


# The context in force; `cache_context(...)` swaps it for the duration of a pipeline call.
_current_cache_context: Optional[CacheContext] = None


def create_cache_context(*args, **kwargs) -> CacheContext:
    return CacheContext(*args, **kwargs)


def get_current_cache_context() -> Optional[CacheContext]:
    return _current_cache_context


def set_current_cache_context(cache_context=None) -> None:
    global _current_cache_context
    _current_cache_context = cache_context


@contextlib.contextmanager
def cache_context(cache_context):
    previous = get_current_cache_context()
    set_current_cache_context(cache_context)
    try:
        yield
    finally:
        set_current_cache_context(previous)


def _ctx() -> CacheContext:
    ctx = get_current_cache_context()
    assert ctx is not None, "cache_context must be set before"
    return ctx


# Module-level accessors of the reference (utils.py:123-217); each acts on the context in force.
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


# Like the reference's (utils.py:123-190), the accessors stay outside compiled regions: they
# read and write Python state that a tracing compiler must not bake into a graph.
for _name in ("get_residual_diff_threshold", "get_buffer", "set_buffer", "remove_buffer", "mark_step_begin",
              "is_taylorseer_enabled", "get_taylorseer", "is_slg_enabled", "slg_should_skip_block", "is_in_warmup",
              "get_downsample_factor"):
    globals()[_name] = torch.compiler.disable(globals()[_name])
del _name


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


@torch.compiler.disable
def fused_residual_diff(h1: torch.Tensor, h0: Optional[torch.Tensor], prev: Optional[torch.Tensor], *,
                        downsample: int = 1, store: bool = True):
    """One launch: ``cur = h1 - h0`` (rounded to the tensors' dtype, optionally only every
    ``downsample``-th channel; ``h0 = None`` means ``cur = h1``), and if ``prev`` is given the fp32
    sums / rounded means / rounded ratio of ``are_two_tensors_similar(prev, cur)``
    (src/para_attn/first_block_cache/utils.py:228-233).

    Returns ``(cur or None, result)`` with ``result`` a 5-float device tensor
    [sum|prev-cur|, sum|prev|, mean_diff, mean_prev, mean_diff/mean_prev]."""
    _require_cuda(h1)
    assert h0 is None or (h1.shape == h0.shape and h1.dtype == h0.dtype)
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
        h1.data_ptr(), h0.data_ptr() if h0 is not None else None, prev.data_ptr() if prev is not None else None,
        cur.data_ptr() if cur is not None else None, rows, cols, downsample, _DTYPES[h1.dtype], result.data_ptr(),
        _scratch_for(h1.device).data_ptr(), torch.cuda.current_stream(h1.device).cuda_stream))
    return cur, result


@torch.compiler.disable
def _axpy(a: torch.Tensor, b: torch.Tensor, sub: bool) -> torch.Tensor:
    """``a - b`` / ``a + b`` rounded to the tensors' 16-bit type: one launch of pa_fbc_axpy (any
    size and 2-byte alignment; sizes that are not a multiple of 8 take its scalar form)."""
    _require_cuda(a)
    if not (_kernel_ok(a, b) and a.shape == b.shape):
        raise NotImplementedError(
            f"cached residual arithmetic needs two contiguous CUDA bf16/f16 tensors of one shape and dtype, got "
            f"{a.dtype} {tuple(a.shape)} and {b.dtype} {tuple(b.shape)}")
    out = torch.empty_like(a)
    if a.numel() > 0:
        L.check(L.load().pa_fbc_axpy(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), 1 if sub else 0,
                                     _DTYPES[a.dtype], torch.cuda.current_stream(a.device).cuda_stream))
    return out


@torch.compiler.disable
def _decide(result: torch.Tensor, dtype: torch.dtype, threshold: float, parallelized: bool) -> bool:
    if parallelized:
        # the reference averages each rounded mean over the default group (utils.py:230-232)
        means = result[2:4].to(dtype)
        means = DP.all_reduce_sync(means, "avg")
        diff = means[0] / means[1]
    else:
        diff = result[4]
    return diff.item() < threshold


@torch.compiler.disable
def are_two_tensors_similar(t1, t2, *, threshold, parallelized=False):
    """mean|t1 - t2| / mean|t1| < threshold with the reference's rounding (utils.py:220-234)."""
    if threshold <= 0.0:
        return False
    if t1.shape != t2.shape:
        return False
    _require_cuda(t1)
    _, result = fused_residual_diff(t2.contiguous(), None, t1.contiguous(), store=False)
    return _decide(result, t1.dtype, threshold, parallelized)


@torch.compiler.disable
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


def _every_nth_channel(residual: torch.Tensor, contiguous: bool = False) -> torch.Tensor:
    """The view of a first-block residual the decision looks at: every ``downsample_factor``-th channel."""
    factor = get_downsample_factor()
    if factor <= 1:
        return residual
    view = residual[..., ::factor]
    return view.contiguous() if contiguous else view


@torch.compiler.disable
def get_can_use_cache(first_hidden_states_residual, parallelized=False):
    """Reference-shaped entry (utils.py:269-286) for callers that already hold the residual:
    no reuse during warm-up, with a threshold of zero, or before a first residual exists."""
    threshold = get_residual_diff_threshold()
    if is_in_warmup() or threshold <= 0.0:
        return False
    previous = get_first_hidden_states_residual()
    if previous is None:
        return False
    return are_two_tensors_similar(previous, _every_nth_channel(first_hidden_states_residual), threshold=threshold,
                                   parallelized=parallelized)


@torch.compiler.disable
def set_first_hidden_states_residual(first_hidden_states_residual):
    set_buffer("first_hidden_states_residual", _every_nth_channel(first_hidden_states_residual, contiguous=True))


def get_first_hidden_states_residual():
    return get_buffer("first_hidden_states_residual")


@torch.compiler.disable
def set_hidden_states_residual(hidden_states_residual):
    """Keep the residual of the skipped blocks: as a buffer, or as a new sample of the extrapolator."""
    if is_taylorseer_enabled():
        get_taylorseer().update(hidden_states_residual)
        return
    set_buffer("hidden_states_residual", hidden_states_residual)


@torch.compiler.disable
def get_hidden_states_residual():
    if is_taylorseer_enabled():
        return get_taylorseer().approximate_value()
    return get_buffer("hidden_states_residual")


def set_encoder_hidden_states_residual(encoder_hidden_states_residual):
    # under TaylorSeer only the hidden states are extrapolated; the encoder states pass through
    if not is_taylorseer_enabled():
        set_buffer("encoder_hidden_states_residual", encoder_hidden_states_residual)


def get_encoder_hidden_states_residual():
    return get_buffer("encoder_hidden_states_residual")


@torch.compiler.disable
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
    """Stands in for a transformer's block list (src/para_attn/first_block_cache/utils.py:333-451):
    runs the first block, decides from its residual whether the rest can be skipped, and either
    applies the cached residual or runs the remaining blocks and caches theirs.

    Blocks take ``(hidden_states, encoder_hidden_states, ...)`` and return a tensor or a pair - in
    the order given by ``return_hidden_states_first`` - which is also what this module returns
    (``return_hidden_states_only`` drops the encoder states). ``single_transformer_blocks`` work on
    the concatenation [encoder states, hidden states] along the sequence."""

    def __init__(self, transformer_blocks, single_transformer_blocks=None, *, transformer=None,
                 return_hidden_states_first=True, return_hidden_states_only=False):
        super().__init__()
        self.transformer = transformer
        self.transformer_blocks = transformer_blocks
        self.single_transformer_blocks = single_transformer_blocks
        self.return_hidden_states_first = return_hidden_states_first
        self.return_hidden_states_only = return_hidden_states_only

    # -- block calling conventions ------------------------------------------------------------
    def _unpack(self, result, encoder_hidden_states):
        """(hidden, encoder) from what a block returned; a bare tensor leaves the encoder states as they were."""
        if isinstance(result, torch.Tensor):
            return result, encoder_hidden_states
        first, second = result
        return (first, second) if self.return_hidden_states_first else (second, first)

    def _pack(self, hidden_states, encoder_hidden_states):
        if self.return_hidden_states_only:
            return hidden_states
        if self.return_hidden_states_first:
            return hidden_states, encoder_hidden_states
        return encoder_hidden_states, hidden_states

    def _is_parallelized(self) -> bool:
        return self.transformer is not None and getattr(self.transformer, "_is_parallelized", False)

    # -- one transformer forward ------------------------------------------------------------------
    def forward(self, hidden_states, encoder_hidden_states, *args, **kwargs):
        block_input = hidden_states
        hidden_states, encoder_hidden_states = self._unpack(
            self.transformer_blocks[0](hidden_states, encoder_hidden_states, *args, **kwargs), encoder_hidden_states)

        mark_step_begin()
        reuse = first_block_decision(hidden_states, block_input, parallelized=self._is_parallelized())
        del block_input

        if reuse:
            hidden_states, encoder_hidden_states = apply_prev_hidden_states_residual(hidden_states,
                                                                                     encoder_hidden_states)
        else:
            hidden_states, encoder_hidden_states, residual, encoder_residual = \
                self.call_remaining_transformer_blocks(hidden_states, encoder_hidden_states, *args, **kwargs)
            set_hidden_states_residual(residual)
            set_encoder_hidden_states_residual(encoder_residual)
        return self._pack(hidden_states, encoder_hidden_states)

    def call_remaining_transformer_blocks(self, hidden_states, encoder_hidden_states, *args, **kwargs):
        """Blocks 1.. of the joint list, then the single-stream list; returns the new states and
        their residuals against the states this method was entered with (utils.py:402-451)."""
        entry_hidden, entry_encoder = hidden_states, encoder_hidden_states
        skip = slg_should_skip_block if is_slg_enabled() else (lambda index: False)
        n_joint = len(self.transformer_blocks)

        for index in range(1, n_joint):
            if skip(index):
                continue
            out = self.transformer_blocks[index](hidden_states, encoder_hidden_states, *args, **kwargs)
            hidden_states, encoder_hidden_states = self._unpack(out, encoder_hidden_states)

        if self.single_transformer_blocks is not None:
            n_text = encoder_hidden_states.shape[1]
            joint = torch.cat([encoder_hidden_states, hidden_states], dim=1)
            for offset, block in enumerate(self.single_transformer_blocks):
                if not skip(n_joint + offset):
                    joint = block(joint, *args, **kwargs)
            encoder_hidden_states, hidden_states = joint.split([n_text, joint.shape[1] - n_text], dim=1)

        def settle(states, entry):
            # a dense copy in the entry tensor's shape (the split above hands out strided views),
            # and the residual against the entry states in the same launch-sized pass
            states = states.reshape(-1).contiguous().reshape(entry.shape)
            return states, _axpy(states, entry.contiguous(), sub=True)

        hidden_states, residual = settle(hidden_states, entry_hidden)
        encoder_residual = None
        if encoder_hidden_states is not None:
            encoder_hidden_states, encoder_residual = settle(encoder_hidden_states, entry_encoder)
        return hidden_states, encoder_hidden_states, residual, encoder_residual
