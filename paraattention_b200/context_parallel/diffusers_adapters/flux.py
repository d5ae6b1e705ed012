"""Context parallelism for FLUX-shaped transformers
(src/para_attn/context_parallel/diffusers_adapters/flux.py:12-109).

Touches: ``transformer.forward(hidden_states, encoder_hidden_states, *args, timestep, img_ids,
txt_ids, controlnet_block_samples, controlnet_single_block_samples, **kwargs)`` whose result's
``[0]`` is the sample, and ``transformer.device``. Image and text tokens are sharded along the
sequence, the blocks run under ``UnifiedAttnMode`` and the sample is gathered at the exit.
"""
import functools
from typing import List, Optional

import torch

from ... import primitives as DP
from ...para_attn_interface import UnifiedAttnMode
from ._common import meshes, patch_pipe_call_for_shared_seed


def parallelize_transformer(transformer, *, mesh=None):
    if getattr(transformer, "_is_parallelized", False):
        return transformer

    mesh, batch_mesh, seq_mesh = meshes(transformer, mesh)
    attn_mode = UnifiedAttnMode(mesh)
    original_forward = transformer.forward

    @functools.wraps(transformer.__class__.forward)
    def new_forward(
        self,
        hidden_states: torch.Tensor,
        encoder_hidden_states: Optional[torch.Tensor] = None,
        *args,
        timestep: torch.LongTensor = None,
        img_ids: torch.Tensor = None,
        txt_ids: torch.Tensor = None,
        controlnet_block_samples: Optional[List[torch.Tensor]] = None,
        controlnet_single_block_samples: Optional[List[torch.Tensor]] = None,
        **kwargs,
    ):
        def shard(x):
            x = DP.get_assigned_chunk(x, dim=0, group=batch_mesh)
            return DP.get_assigned_chunk(x, dim=-2, group=seq_mesh)

        if isinstance(timestep, torch.Tensor) and timestep.ndim != 0 and timestep.shape[0] == hidden_states.shape[0]:
            timestep = DP.get_assigned_chunk(timestep, dim=0, group=batch_mesh)
        hidden_states = shard(hidden_states)
        encoder_hidden_states = shard(encoder_hidden_states)
        # the reference chunks the position ids over the default group (flux.py:41-42)
        img_ids = DP.get_assigned_chunk(img_ids, dim=-2)
        txt_ids = DP.get_assigned_chunk(txt_ids, dim=-2)
        if controlnet_block_samples is not None:
            kwargs["controlnet_block_samples"] = [shard(s) for s in controlnet_block_samples]
        if controlnet_single_block_samples is not None:
            kwargs["controlnet_single_block_samples"] = [shard(s) for s in controlnet_single_block_samples]

        with attn_mode:
            output = original_forward(
                hidden_states,
                encoder_hidden_states,
                *args,
                timestep=timestep,
                img_ids=img_ids,
                txt_ids=txt_ids,
                **kwargs,
            )

        return_dict = not isinstance(output, tuple)
        sample = output[0]
        sample = DP.get_complete_tensor(sample, dim=-2, group=seq_mesh)
        sample = DP.get_complete_tensor(sample, dim=0, group=batch_mesh)
        if return_dict:
            return output.__class__(sample, *output[1:])
        return (sample, *output[1:])

    transformer.forward = new_forward.__get__(transformer)
    transformer._is_parallelized = True
    return transformer


def parallelize_pipe(pipe, *, shallow_patch: bool = False, **kwargs):
    patch_pipe_call_for_shared_seed(pipe)
    if not shallow_patch:
        parallelize_transformer(pipe.transformer, **kwargs)
    return pipe
