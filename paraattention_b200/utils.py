"""Helpers shared by the attention modes (src/para_attn/utils.py:12-32)."""
import torch
from packaging.version import parse as _parse_version
from torch.overrides import TorchFunctionMode

from . import config


def torch_version_check(op: str, v: str) -> bool:
    """``torch_version_check("__ge__", "2.6.0")``: compare the running torch version with ``v``."""
    compare = getattr(_parse_version(torch.__version__), op)
    return compare(_parse_version(v))


@torch.compiler.assume_constant_result
def get_force_dispatch_to_custom_ops() -> bool:
    # read at trace time as a constant, like every other configuration switch
    return bool(config.attention.force_dispatch_to_custom_ops)


@torch.compiler.assume_constant_result
def get_allow_sdpa_fallback() -> bool:
    return bool(config.attention.allow_sdpa_fallback)


class BaseTorchFunctionMode(TorchFunctionMode):
    """TorchFunctionMode whose construction stays outside compiled regions."""

    @torch.compiler.disable
    def __init__(self):
        super().__init__()


def base_handle_torch_function(func, types, args=(), kwargs=None):
    """Run ``func`` as if no mode were active. ``Tensor.unflatten`` reaches its implementation
    through ``super()``, which the function-mode machinery cannot re-dispatch, so it is swapped for
    the equivalent free function (src/para_attn/utils.py:28-30)."""
    call = torch.unflatten if func is torch.Tensor.unflatten else func
    return call(*args, **(kwargs or {}))
