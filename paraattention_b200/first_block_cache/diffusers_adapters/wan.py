"""First Block Cache for Wan-shaped transformers
(src/para_attn/first_block_cache/diffusers_adapters/wan.py:10-79): ``blocks`` return hidden
states only; the pipeline runs the transformer twice per step (conditional / unconditional),
so the alternate cache is on by default and ``num_inference_steps`` defaults to 50."""
from .. import utils
from ._common import install_cached_forward, single, wrap_pipe_call


def apply_cache_on_transformer(transformer):
    if getattr(transformer, "_is_cached", False):
        return transformer
    cached = single(
        utils.CachedTransformerBlocks(transformer.blocks, transformer=transformer, return_hidden_states_only=True))
    return install_cached_forward(transformer, {"blocks": cached})


def apply_cache_on_pipe(pipe, *, shallow_patch: bool = False, enable_alter_cache: bool = True, **kwargs):
    def make_context():
        kw = dict(kwargs)
        kw.setdefault("num_inference_steps", 50)
        return utils.create_cache_context(enable_alter_cache=enable_alter_cache, **kw)

    wrap_pipe_call(pipe, make_context)
    if not shallow_patch:
        apply_cache_on_transformer(pipe.transformer)
    return pipe
