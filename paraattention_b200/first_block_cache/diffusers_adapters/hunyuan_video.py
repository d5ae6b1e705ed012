"""First Block Cache for HunyuanVideo-shaped transformers
(src/para_attn/first_block_cache/diffusers_adapters/hunyuan_video.py:16-206): the dual-stream
and single-stream blocks share one signature and return (hidden_states,
encoder_hidden_states), so they are chained in ONE list. The model's own forward (or the
context-parallel forward installed by ``parallelize_transformer``) runs unchanged around it."""
import torch

from .. import utils
from ._common import install_cached_forward, single, wrap_pipe_call


def apply_cache_on_transformer(transformer):
    if getattr(transformer, "_is_cached", False):
        return transformer
    chained = torch.nn.ModuleList(list(transformer.transformer_blocks) + list(transformer.single_transformer_blocks))
    cached = single(utils.CachedTransformerBlocks(chained, transformer=transformer))
    return install_cached_forward(
        transformer, {"transformer_blocks": cached, "single_transformer_blocks": torch.nn.ModuleList()})


def apply_cache_on_pipe(pipe, *, shallow_patch: bool = False, **kwargs):
    wrap_pipe_call(pipe, lambda: utils.create_cache_context(**kwargs))
    if not shallow_patch:
        apply_cache_on_transformer(pipe.transformer)
    return pipe
