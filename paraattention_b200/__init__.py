"""B200-native context-parallel attention engine with the ParaAttention API surface.

The compute path is the CUDA library ``libpa_b200.so`` (hand-written sm_100a kernels behind a
C ABI, see ``include/pa_b200.h``); this package is the host-side mirror of the reference's
Python interface for that path (src/para_attn/__init__.py:8-26). There is no CPU or PyTorch
fallback for the kernels: importing works anywhere, calling an op without the built
library or without a CUDA device raises.

``install_as_para_attn()`` registers this package under the name ``para_attn`` so that code
written against the reference (``import para_attn``; ``from para_attn.context_parallel
import ...``) runs unchanged.
"""
import importlib
import sys

__version__ = "0.1.0"

from . import config, ops  # noqa: E402
from .para_attn_interface import (  # noqa: E402
    in_batch_attn_func,
    InBatchAttnMode,
    ring_attn_func,
    RingAttnMode,
    sparse_kv_attn_func,
    SparseKVAttnMode,
    ulysses_attn_func,
    UlyssesAttnMode,
    UnifiedAttnMode,
)
from ._cp_engine import check_device_status, reset_device_status  # noqa: E402
from .host_io import attention_from_host  # noqa: E402

__all__ = [
    "UnifiedAttnMode",
    "RingAttnMode",
    "UlyssesAttnMode",
    "InBatchAttnMode",
    "SparseKVAttnMode",
    "sparse_kv_attn_func",
    "ring_attn_func",
    "ulysses_attn_func",
    "in_batch_attn_func",
    "check_device_status",
    "reset_device_status",
    "attention_from_host",
    "install_as_para_attn",
]

_SUBMODULES = (
    "config", "ops", "primitives", "utils", "para_attn_interface", "sparse_attn",
    "context_parallel", "context_parallel.diffusers_adapters",
    "first_block_cache", "first_block_cache.utils", "first_block_cache.diffusers_adapters",
)


def install_as_para_attn() -> None:
    """Alias this package (and its submodules) as ``para_attn`` in ``sys.modules``."""
    if "para_attn" in sys.modules and sys.modules["para_attn"] is not sys.modules[__name__]:
        raise RuntimeError("another package named para_attn is already imported")
    sys.modules["para_attn"] = sys.modules[__name__]
    for sub in _SUBMODULES:
        mod = importlib.import_module(f"{__name__}.{sub}")
        sys.modules[f"para_attn.{sub}"] = mod
