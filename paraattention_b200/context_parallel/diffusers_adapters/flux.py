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
    unsharded_forward = transformer.forward

    def of_my_batch(x):
        return DP.get_assigned_chunk(x, dim=0, group=batch_mesh)

    def shard(x):
        """Batch entries of this rank, then its piece of the sequence."""
        return DP.get_assigned_chunk(of_my_batch(x), dim=-2, group=seq_mesh)

    def gather(x):
        x = DP.get_complete_tensor(x, dim=-2, group=seq_mesh)
        return DP.get_complete_tensor(x, dim=0, group=batch_mesh)

    @functools.wraps(transformer.__class__.forward)
    def new_forward(self, hidden_states: torch.Tensor, encoder_hidden_states: Optional[torch.Tensor] = None, *args,
                    timestep: torch.LongTensor = None, img_ids: torch.Tensor = None, txt_ids: torch.Tensor = None,
                    controlnet_block_samples: Optional[List[torch.Tensor]] = None,
                    controlnet_single_block_samples: Optional[List[torch.Tensor]] = None, **kwargs):
        per_sample_timestep = (isinstance(timestep, torch.Tensor) and timestep.ndim != 0
                               and timestep.shape[0] == hidden_states.shape[0])
        if per_sample_timestep:
            timestep = of_my_batch(timestep)
        # residuals injected by a ControlNet follow the tokens they are added to
        for name, samples in (("controlnet_block_samples", controlnet_block_samples),
                              ("controlnet_single_block_samples", controlnet_single_block_samples)):
            if samples is not None:
                kwargs[name] = [shard(sample) for sample in samples]

        with attn_mode:
            output = unsharded_forward(
                shard(hidden_states), shard(encoder_hidden_states), *args, timestep=timestep,
                # the position ids carry no batch dimension: the reference splits them over the
                # default group (flux.py:41-42)
                img_ids=DP.get_assigned_chunk(img_ids, dim=-2), txt_ids=DP.get_assigned_chunk(txt_ids, dim=-2),
                **kwargs)

        # the sample is element 0 of a tuple or of a model-output object; everything else passes through
        sample, rest = gather(output[0]), tuple(output[1:])
        if isinstance(output, tuple):
            return (sample,) + rest
        return output.__class__(sample, *rest)

    transformer.forward = new_forward.__get__(transformer)
    transformer._is_parallelized = True
    return transformer


def parallelize_pipe(pipe, *, shallow_patch: bool = False, **kwargs):
    """Patch the pipeline's call (shared seed) and, unless ``shallow_patch``, its transformer."""
    patch_pipe_call_for_shared_seed(pipe)
    if shallow_patch:
        return pipe
    parallelize_transformer(pipe.transformer, **kwargs)
    return pipe
