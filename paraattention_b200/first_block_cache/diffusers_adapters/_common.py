"""Shared mechanics of the cache adapters: swapping a transformer's block lists for one
``CachedTransformerBlocks`` while its forward runs, and giving every pipeline call a fresh
``CacheContext`` (the reference does both per model file, e.g.
src/para_attn/first_block_cache/diffusers_adapters/flux.py:10-77)."""
import contextlib
import functools

import torch

from .. import utils


@contextlib.contextmanager
def swapped_attributes(obj, **replacements):
    """Temporarily replace attributes of ``obj`` (restored even if the body raises)."""
    saved = {name: getattr(obj, name) for name in replacements}
    try:
        for name, value in replacements.items():
            setattr(obj, name, value)
        yield
    finally:
        for name, value in saved.items():
            setattr(obj, name, value)


def install_cached_forward(transformer, replacements):
    """Wrap ``transformer.forward`` so that ``replacements`` (attribute name -> module list) are
    in place for the duration of each call. Idempotent through ``_is_cached``."""
    original_forward = transformer.forward

    @functools.wraps(transformer.__class__.forward)
    def new_forward(self, *args, **kwargs):
        with swapped_attributes(self, **replacements):
            return original_forward(*args, **kwargs)

    transformer.forward = new_forward.__get__(transformer)
    transformer._is_cached = True
    return transformer


def wrap_pipe_call(pipe, make_context):
    """Class-level patch of ``__call__``: each pipeline call runs inside a new cache context."""
    if getattr(pipe, "_is_cached", False):
        return
    original_call = pipe.__class__.__call__

    @functools.wraps(original_call)
    def new_call(self, *args, **kwargs_):
        with utils.cache_context(make_context()):
            return original_call(self, *args, **kwargs_)

    pipe.__class__.__call__ = new_call
    pipe.__class__._is_cached = True


def single(module) -> torch.nn.ModuleList:
    return torch.nn.ModuleList([module])
