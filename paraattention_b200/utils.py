"""Helpers shared by the attention modes (src/para_attn/utils.py:12-32)."""
import torch
from packaging import version
from torch.overrides import TorchFunctionMode

from . import config


def torch_version_check(op, v):
    return getattr(version.parse(torch.__version__), op)(version.parse(v))


@torch.compiler.assume_constant_result
def get_force_dispatch_to_custom_ops():
    return config.attention.force_dispatch_to_custom_ops


class BaseTorchFunctionMode(TorchFunctionMode):
    @torch.compiler.disable
    def __init__(self):
        super().__init__()


def base_handle_torch_function(func, types, args=(), kwargs=None):
    kwargs = {} if kwargs is None else kwargs
    if func is torch.Tensor.unflatten:
        # Tensor.unflatten reaches its implementation through super(), which the function-mode
        # machinery cannot re-dispatch; the free function is equivalent (src/para_attn/utils.py:28-30)
        return torch.unflatten(*args, **kwargs)
    return func(*args, **kwargs)
