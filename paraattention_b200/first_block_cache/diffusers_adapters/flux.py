"""First Block Cache for FLUX-shaped transformers
(src/para_attn/first_block_cache/diffusers_adapters/flux.py:10-77): the dual-stream and the
single-stream block lists become one ``CachedTransformerBlocks`` (blocks return
(encoder_hidden_states, hidden_states), hence ``return_hidden_states_first=False``)."""
import torch

from .. import utils
from ._common import install_cached_forward, single, wrap_pipe_call


def apply_cache_on_transformer(transformer):
    if getattr(transformer, "_is_cached", False):
        return transformer
    cached = single(
        utils.CachedTransformerBlocks(
            transformer.transformer_blocks,
            transformer.single_transformer_blocks,
            transformer=transformer,
            return_hidden_states_first=False,
        )
    )
    return install_cached_forward(
        transformer, {"transformer_blocks": cached, "single_transformer_blocks": torch.nn.ModuleList()})


def apply_cache_on_pipe(pipe, *, shallow_patch: bool = False, **kwargs):
    wrap_pipe_call(pipe, lambda: utils.create_cache_context(**kwargs))
    if not shallow_patch:
        apply_cache_on_transformer(pipe.transformer)
    return pipe
