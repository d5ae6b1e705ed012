"""``apply_cache_on_pipe`` / ``apply_cache_on_transformer``: dispatch on the class-name prefix
like the reference (src/para_attn/first_block_cache/diffusers_adapters/__init__.py:6-49).
Adapters exist for the model families of the accelerated path: Flux, Wan, HunyuanVideo."""
import importlib

_ADAPTERS = (("Flux", "flux"), ("HunyuanVideo", "hunyuan_video"), ("Wan", "wan"))
_NOT_BUILT = ("Mochi", "CogVideoX")


def _adapter_for(cls_name: str, what: str):
    for prefix, name in _ADAPTERS:
        if cls_name.startswith(prefix):
            return importlib.import_module(f".{name}", __package__)
    for prefix in _NOT_BUILT:
        if cls_name.startswith(prefix):
            raise NotImplementedError(f"{what} class {cls_name}: no adapter for {prefix} models in this package")
    raise ValueError(f"Unknown {what} class name: {cls_name}")


def apply_cache_on_transformer(transformer, *args, **kwargs):
    module = _adapter_for(transformer.__class__.__name__, "transformer")
    return module.apply_cache_on_transformer(transformer, *args, **kwargs)


def apply_cache_on_pipe(pipe, *args, **kwargs):
    try:
        from diffusers import DiffusionPipeline

        assert isinstance(pipe, DiffusionPipeline)
    except ImportError:
        pass  # duck-typed pipelines are accepted where diffusers is not installed
    module = _adapter_for(pipe.__class__.__name__, "pipeline")
    return module.apply_cache_on_pipe(pipe, *args, **kwargs)
