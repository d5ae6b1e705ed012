"""Runtime switches with the reference's names (src/para_attn/config.py:12-29).

``attention.force_dispatch_to_custom_ops``: in the reference it routes the final,
non-parallel SDPA of ``UnifiedAttnMode`` through the custom op instead of
``F.scaled_dot_product_attention``. Here the custom op *is* the product path; the flag is kept
for code that sets it and changes nothing.

``attention.allow_sdpa_fallback`` (no counterpart in the reference): an attention call inside a
mode that the sm_100a kernel does not cover raises; with this set it goes to PyTorch's own
SDPA instead. Off by default: nothing leaves the kernel path silently.

``attention.allow_reduced_precision_compute``: the reference lets torch's ring merger run in
the block dtype when set. The fused kernel always accumulates and merges in fp32 on chip,
so both settings produce the fp32-merge result.
"""
import os
import sys


class attention:
    force_dispatch_to_custom_ops = os.getenv("PARA_ATTN_FORCE_DISPATCH_TO_CUSTOM_OPS") == "1"
    allow_reduced_precision_compute = os.getenv("PARA_ATTN_ALLOW_REDUCED_PRECISION_COMPUTE") == "1"
    allow_sdpa_fallback = os.getenv("PA_B200_ALLOW_SDPA_FALLBACK") == "1"
    # the shape-only transformers of this package prepare q, k, v with the fused kernel
    # (ops.qkv_prepare) instead of a chain of tensor operations when their tensors allow it
    fuse_qkv_prepare = os.getenv("PA_B200_FUSE_QKV_PREPARE", "1") == "1"
    # non-causal single-GPU attention launches whose last wave of CTAs would leave most SMs idle
    # give the work units of that wave to several CTAs each (the keys are split among them; the
    # library decides per shape). Costs one scratch buffer of 64 MB per device and stream.
    # Context-parallel launches never do this (measured slower with real peers).
    split_last_wave = os.getenv("PA_B200_SPLIT_LAST_WAVE", "1") == "1"


class cp:
    """Knobs of the NVLink exchange that have no counterpart in the reference."""

    # how many leading CTAs of the attention grid do the exchange (0 = choose from the bytes to send)
    push_ctas_per_dest = int(os.getenv("PA_B200_PUSH_CTAS", "0"))
    # get_complete_tensor (the gather at the exit of a parallelised forward) as peer stores
    peer_gather = os.getenv("PA_B200_PEER_GATHER", "1") == "1"
    # Ulysses output: hand out the staging buffer itself instead of a private copy. The tensor is
    # then overwritten by the second-next attention call of the same mesh: only for callers that
    # consume an attention result before issuing two more (every transformer block does).
    zero_copy_output = os.getenv("PA_B200_ZERO_COPY_OUTPUT") == "1"
    # device-side bound on every wait for a peer, in nanoseconds
    wait_limit_ns = int(os.getenv("PA_B200_WAIT_LIMIT_NS", str(5_000_000_000)))


from torch.utils._config_module import install_config_module  # noqa: E402

# adds patch(), save_config(), ... exactly like the reference's module
install_config_module(sys.modules[__name__])
