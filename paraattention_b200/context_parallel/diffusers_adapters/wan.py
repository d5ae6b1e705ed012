"""Context parallelism for Wan-shaped transformers
(src/para_attn/context_parallel/diffusers_adapters/wan.py:17-168).

The forward is re-stated from the attributes the reference uses: ``config.patch_size``,
``rope``, ``patch_embedding``, ``condition_embedder``, ``blocks``, ``scale_shift_table``,
``norm_out``, ``proj_out``. Video tokens and their rotary table are sharded along the
sequence; the text states are sharded over the batch only, so every rank's cross-attention
keys are the full prompt (replicated keys leave softmax attention unchanged).
"""
import functools
from typing import Any, Dict, Optional, Union

import torch

from ... import primitives as DP
from ...para_attn_interface import UnifiedAttnMode
from ._common import make_output, meshes, patch_pipe_call_for_shared_seed


def parallelize_transformer(transformer, *, mesh=None):
    if getattr(transformer, "_is_parallelized", False):
        return transformer

    mesh, batch_mesh, seq_mesh = meshes(transformer, mesh)
    attn_mode = UnifiedAttnMode(mesh)

    @functools.wraps(transformer.__class__.forward)
    def new_forward(
        self,
        hidden_states: torch.Tensor,
        timestep: torch.LongTensor,
        encoder_hidden_states: torch.Tensor,
        encoder_hidden_states_image: Optional[torch.Tensor] = None,
        return_dict: bool = True,
        attention_kwargs: Optional[Dict[str, Any]] = None,
        **kwargs,
    ) -> Union[torch.Tensor, Dict[str, torch.Tensor]]:
        batch_size, num_channels, num_frames, height, width = hidden_states.shape
        p_t, p_h, p_w = self.config.patch_size
        post_patch_num_frames = num_frames // p_t
        post_patch_height = height // p_h
        post_patch_width = width // p_w

        rotary_emb = self.rope(hidden_states)

        hidden_states = self.patch_embedding(hidden_states)
        hidden_states = hidden_states.flatten(2).transpose(1, 2)

        temb, timestep_proj, encoder_hidden_states, encoder_hidden_states_image = self.condition_embedder(
            timestep, encoder_hidden_states, encoder_hidden_states_image
        )
        timestep_proj = timestep_proj.unflatten(1, (6, -1))

        if encoder_hidden_states_image is not None:
            encoder_hidden_states = torch.concat([encoder_hidden_states_image, encoder_hidden_states], dim=1)

        timestep_proj = DP.get_assigned_chunk(timestep_proj, dim=0, group=batch_mesh)
        temb = DP.get_assigned_chunk(temb, dim=0, group=batch_mesh)
        hidden_states = DP.get_assigned_chunk(hidden_states, dim=0, group=batch_mesh)
        hidden_states = DP.get_assigned_chunk(hidden_states, dim=-2, group=seq_mesh)
        encoder_hidden_states = DP.get_assigned_chunk(encoder_hidden_states, dim=0, group=batch_mesh)
        # the rotary table is shared by the batch: shard it along the sequence only
        rotary_emb = DP.get_assigned_chunk(rotary_emb, dim=-2, group=seq_mesh)

        with attn_mode:
            hidden_states = self.call_transformer_blocks(hidden_states, encoder_hidden_states, timestep_proj, rotary_emb)

        shift, scale = (self.scale_shift_table + temb.unsqueeze(1)).chunk(2, dim=1)
        hidden_states = (self.norm_out(hidden_states.float()) * (1 + scale) + shift).type_as(hidden_states)
        hidden_states = self.proj_out(hidden_states)

        hidden_states = DP.get_complete_tensor(hidden_states, dim=-2, group=seq_mesh)
        hidden_states = DP.get_complete_tensor(hidden_states, dim=0, group=batch_mesh)

        hidden_states = hidden_states.reshape(
            batch_size, post_patch_num_frames, post_patch_height, post_patch_width, p_t, p_h, p_w, -1
        )
        hidden_states = hidden_states.permute(0, 7, 1, 4, 2, 5, 3, 6)
        output = hidden_states.flatten(6, 7).flatten(4, 5).flatten(2, 3)
        return make_output(getattr(self, "output_class", None), output, return_dict)

    transformer.forward = new_forward.__get__(transformer)

    def call_transformer_blocks(self, hidden_states, encoder_hidden_states, *args, **kwargs):
        for block in self.blocks:
            hidden_states = block(hidden_states, encoder_hidden_states, *args, **kwargs)
        return hidden_states

    transformer.call_transformer_blocks = call_transformer_blocks.__get__(transformer)
    transformer._is_parallelized = True
    return transformer


def parallelize_pipe(pipe, *, shallow_patch: bool = False, **kwargs):
    patch_pipe_call_for_shared_seed(pipe)
    if not shallow_patch:
        parallelize_transformer(pipe.transformer, **kwargs)
    return pipe
