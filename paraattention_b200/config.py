"""Runtime switches with the reference's names (src/para_attn/config.py:12-29).

``attention.force_dispatch_to_custom_ops``: in the reference it routes the final,
non-parallel SDPA of ``UnifiedAttnMode`` through the custom op instead of
``F.scaled_dot_product_attention``. Here the custom op *is* the product path, so the CUDA
bf16/f16 head_dim 64 / 128 case always goes to it; the flag additionally makes unsupported
inputs raise instead of being handed back to PyTorch's own SDPA.

``attention.allow_reduced_precision_compute``: the reference lets torch's ring merger run in
the block dtype when set. The fused kernel always accumulates and merges in fp32 on chip,
so both settings produce the fp32-merge result.
"""
import os
import sys


class attention:
    force_dispatch_to_custom_ops = os.getenv("PARA_ATTN_FORCE_DISPATCH_TO_CUSTOM_OPS") == "1"
    allow_reduced_precision_compute = os.getenv("PARA_ATTN_ALLOW_REDUCED_PRECISION_COMPUTE") == "1"


class cp:
    """Knobs of the NVLink exchange that have no counterpart in the reference."""

    # how many leading CTAs of the attention grid do the exchange (0 = choose from the bytes to send)
    push_ctas_per_dest = int(os.getenv("PA_B200_PUSH_CTAS", "0"))
    # device-side bound on every wait for a peer, in nanoseconds
    wait_limit_ns = int(os.getenv("PA_B200_WAIT_LIMIT_NS", str(5_000_000_000)))


from torch.utils._config_module import install_config_module  # noqa: E402

# adds patch(), save_config(), ... exactly like the reference's module
install_config_module(sys.modules[__name__])
