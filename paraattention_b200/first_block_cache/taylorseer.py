"""TaylorSeer: extrapolate the cached residual instead of reusing it unchanged
(src/para_attn/first_block_cache/taylorseer.py:4-64, same constructor, methods and step rules).

Parity note: the quotient ``(d_i - prev_i) / window`` is the correctly rounded IEEE division, which
is what the reference computes on CPU tensors. On CUDA tensors ATen divides by a Python scalar as
``a * (1 / window)``, which for windows that are not powers of two can differ from the true
quotient by one step of the 16-bit type in a rare element; the fixtures pin the CPU result.

On a computed step ``update(Y)`` keeps Y and finite-difference estimates of its derivatives
over the steps since the last computed one; on a skipped step ``approximate_value()`` returns
the Taylor sum at the current step. Where the reference chains tensor operations (two per
derivative, three per term), each call here is one pass of a kernel of libpa_b200 with the same
intermediate roundings, so results are identical bit for bit. CUDA tensors only.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from .. import _lib as L

_DTYPES = {torch.bfloat16: L.PA_BF16, torch.float16: L.PA_F16}
_MAX_DERIVATIVES = 4


def _check(t: torch.Tensor, what: str) -> None:
    if t.device.type != "cuda":
        raise RuntimeError("TaylorSeer kernels need CUDA tensors; there is no CPU path in this package")
    if t.dtype not in _DTYPES or not t.is_contiguous() or t.numel() % 8 != 0 or t.data_ptr() % 16 != 0:
        raise NotImplementedError(f"{what}: expected a contiguous bf16/f16 tensor with a multiple of 8 elements, got "
                                  f"{t.dtype} {tuple(t.shape)}")


class TaylorSeer:
    """Same constructor arguments, public attributes (``ORDER``, ``current_step``,
    ``last_non_approximated_step``, ``state``) and methods as the reference class; the
    bookkeeping below is this package's own, the arithmetic lives in the kernels."""

    def __init__(self, n_derivatives=2, warmup_steps=1, skip_interval_steps=1, compute_step_map=None):
        if n_derivatives > _MAX_DERIVATIVES:
            raise NotImplementedError(f"n_derivatives {n_derivatives}: the kernels hold at most {_MAX_DERIVATIVES}")
        self.n_derivatives = n_derivatives
        self.warmup_steps = warmup_steps
        self.skip_interval_steps = skip_interval_steps
        self.compute_step_map = compute_step_map
        self.reset_cache()

    @property
    def ORDER(self) -> int:
        """Number of Taylor terms: the value itself plus ``n_derivatives`` differences."""
        return self.n_derivatives + 1

    def reset_cache(self):
        # derivative estimates of the last computed step and of the one before it, lowest order first
        self._estimates: List[Optional[torch.Tensor]] = [None] * self.ORDER
        self._older: List[Optional[torch.Tensor]] = [None] * self.ORDER
        self.current_step = -1
        self.last_non_approximated_step = -1

    @property
    def state(self):
        """The reference's view of the two estimate lists (taylorseer.py:13-17)."""
        return {"dY_prev": self._older, "dY_current": self._estimates}

    def should_compute_full(self, step=None):
        """Whether ``step`` (default: the current one) runs the model: an explicit per-step map wins,
        otherwise the warm-up steps and then every ``skip_interval_steps``-th step after them."""
        s = self.current_step if step is None else step
        if self.compute_step_map is not None:
            return self.compute_step_map[s]
        past_warmup = s - self.warmup_steps
        return past_warmup < 0 or (past_warmup + 1) % self.skip_interval_steps == 0

    def approximate_derivative(self, Y: torch.Tensor) -> List[Optional[torch.Tensor]]:
        """d_0 = Y and, as far as the previous computed step has them and two steps have passed,
        d_{i+1} = (d_i - prev_i) / window (taylorseer.py:29-38): one kernel for the whole chain."""
        _check(Y, "TaylorSeer.update")
        fresh: List[Optional[torch.Tensor]] = [None] * self.ORDER
        fresh[0] = Y
        window = self.current_step - self.last_non_approximated_step
        depth = 0
        if self.current_step > 1:
            while depth < self.n_derivatives and self._older[depth] is not None:
                depth += 1
        if depth == 0:
            return fresh
        prev = self._older[:depth]
        for t in prev:
            assert t.shape == Y.shape and t.dtype == Y.dtype, "the residual changed shape or dtype between steps"
        for i in range(depth):
            fresh[i + 1] = torch.empty_like(Y)
        prev_p = (C.c_void_p * depth)(*[t.data_ptr() for t in prev])
        cur_p = (C.c_void_p * depth)(*[fresh[i + 1].data_ptr() for i in range(depth)])
        L.check(L.load().pa_taylor_update(Y.data_ptr(), prev_p, cur_p, depth, window, Y.numel(), _DTYPES[Y.dtype],
                                          torch.cuda.current_stream(Y.device).cuda_stream))
        return fresh

    def approximate_value(self, add: Optional[torch.Tensor] = None):
        """sum_i d_i * elapsed^i / i! over the derivatives at hand (taylorseer.py:40-48). With
        ``add`` the same launch also adds that tensor (the hidden states the residual belongs to)."""
        elapsed = self.current_step - self.last_non_approximated_step
        terms = 0
        while terms < self.ORDER and self._estimates[terms] is not None:
            terms += 1
        if terms == 0:
            return 0 if add is None else add
        d = self._estimates[:terms]
        if add is not None:
            _check(add, "TaylorSeer.approximate_value")
            assert add.shape == d[0].shape and add.dtype == d[0].dtype
        out = torch.empty_like(d[0])
        d_p = (C.c_void_p * terms)(*[t.data_ptr() for t in d])
        L.check(L.load().pa_taylor_approx(d_p, terms, elapsed, add.data_ptr() if add is not None else None,
                                          out.data_ptr(), out.numel(), _DTYPES[out.dtype],
                                          torch.cuda.current_stream(out.device).cuda_stream))
        return out

    def mark_step_begin(self):
        self.current_step += 1

    def update(self, Y):
        """A computed step: the estimates of the last computed step become the older ones (they
        are what the new differences are taken against) and this step becomes the anchor."""
        self._older = self._estimates
        self._estimates = self.approximate_derivative(Y)
        self.last_non_approximated_step = self.current_step

    def step(self, Y):
        """One step of the schedule: the model's output on computed steps, the extrapolation otherwise."""
        self.mark_step_begin()
        if not self.should_compute_full():
            return self.approximate_value()
        self.update(Y)
        return Y
