"""Context parallelism for HunyuanVideo-shaped transformers
(src/para_attn/context_parallel/diffusers_adapters/hunyuan_video.py:16-217).

Attributes used: ``config.patch_size``, ``config.patch_size_t``, ``rope``, ``time_text_embed``,
``x_embedder``, ``context_embedder``, ``transformer_blocks``, ``single_transformer_blocks``,
``norm_out``, ``proj_out``. Video tokens, text tokens and both rotary tables are sharded along
the sequence; each rank's joint sequence is [its video shard, its text shard].

The reference builds a key-padding mask over video + text tokens, re-orders it to that
interleaved layout (:74-100) and lets ``SparseKVAttnMode`` drop padded keys before attention
(:112). Here the mask - in the same interleaved order, one [video shard, text shard] piece per
rank of the sequence mesh - goes into the chunked attention kernel, which also works when the
mesh has a ring dimension. The mask is always passed (an all-true mask costs the kernel nothing
worth a device-to-host round trip to find out), so a forward has no host synchronisation.
PEFT LoRA scaling (``attention_kwargs["scale"]``, :54-67 and :124-126 of the reference) is applied
when diffusers is importable.
"""
import functools
from typing import Any, Dict, Optional, Union

import torch

try:  # LoRA scale handling needs diffusers; the duck-typed stand-ins of this package do not
    from diffusers.utils import scale_lora_layers, unscale_lora_layers, USE_PEFT_BACKEND
except Exception:  # pragma: no cover - diffusers is optional
    scale_lora_layers = unscale_lora_layers = None
    USE_PEFT_BACKEND = False

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
        encoder_attention_mask: torch.Tensor,
        pooled_projections: torch.Tensor,
        guidance: torch.Tensor = None,
        attention_kwargs: Optional[Dict[str, Any]] = None,
        return_dict: bool = True,
        **kwargs,
    ) -> Union[torch.Tensor, Dict[str, torch.Tensor]]:
        lora_scale = 1.0
        if attention_kwargs is not None:
            attention_kwargs = dict(attention_kwargs)
            lora_scale = attention_kwargs.pop("scale", 1.0)
        if USE_PEFT_BACKEND and scale_lora_layers is not None:
            scale_lora_layers(self, lora_scale)

        batch_size, num_channels, num_frames, height, width = hidden_states.shape
        p, p_t = self.config.patch_size, self.config.patch_size_t
        post_patch_num_frames = num_frames // p_t
        post_patch_height = height // p
        post_patch_width = width // p

        image_rotary_emb = self.rope(hidden_states)

        temb = self.time_text_embed(timestep, guidance, pooled_projections)
        hidden_states = self.x_embedder(hidden_states)
        encoder_hidden_states = self.context_embedder(encoder_hidden_states, timestep, encoder_attention_mask)

        prompt_mask = encoder_attention_mask.to(torch.bool)
        world = DP.get_world_size(seq_mesh)
        n_video, n_text = hidden_states.shape[1], encoder_hidden_states.shape[1]
        assert n_video % world == 0 and n_text % world == 0, "sequence lengths must divide by the mesh size"
        video = torch.ones(batch_size, n_video // world, dtype=torch.bool, device=prompt_mask.device)
        pieces = []
        for piece in prompt_mask.chunk(world, dim=-1):
            pieces += [video, piece]
        attention_mask = torch.cat(pieces, dim=-1)[:, None, None, :]
        attention_mask = DP.get_assigned_chunk(attention_mask, dim=0, group=batch_mesh)

        temb = DP.get_assigned_chunk(temb, dim=0, group=batch_mesh)
        hidden_states = DP.get_assigned_chunk(hidden_states, dim=0, group=batch_mesh)
        hidden_states = DP.get_assigned_chunk(hidden_states, dim=-2, group=seq_mesh)
        encoder_hidden_states = DP.get_assigned_chunk(encoder_hidden_states, dim=0, group=batch_mesh)
        encoder_hidden_states = DP.get_assigned_chunk(encoder_hidden_states, dim=-2, group=seq_mesh)

        freqs_cos, freqs_sin = image_rotary_emb
        freqs_cos = DP.get_assigned_chunk(freqs_cos, dim=0, group=seq_mesh)
        freqs_sin = DP.get_assigned_chunk(freqs_sin, dim=0, group=seq_mesh)
        image_rotary_emb = (freqs_cos, freqs_sin)

        with attn_mode:
            hidden_states, encoder_hidden_states = self.call_transformer_blocks(
                hidden_states, encoder_hidden_states, temb, attention_mask, image_rotary_emb
            )

        hidden_states = self.norm_out(hidden_states, temb)
        hidden_states = self.proj_out(hidden_states)

        hidden_states = DP.get_complete_tensor(hidden_states, dim=-2, group=seq_mesh)
        hidden_states = DP.get_complete_tensor(hidden_states, dim=0, group=batch_mesh)

        hidden_states = hidden_states.reshape(
            batch_size, post_patch_num_frames, post_patch_height, post_patch_width, -1, p_t, p, p
        )
        hidden_states = hidden_states.permute(0, 4, 1, 5, 2, 6, 3, 7)
        hidden_states = hidden_states.flatten(6, 7).flatten(4, 5).flatten(2, 3)
        if isinstance(timestep, torch.Tensor) and timestep.is_floating_point():
            hidden_states = hidden_states.to(timestep.dtype)
        if USE_PEFT_BACKEND and unscale_lora_layers is not None:
            unscale_lora_layers(self, lora_scale)
        return make_output(getattr(self, "output_class", None), hidden_states, return_dict)

    transformer.forward = new_forward.__get__(transformer)

    def call_transformer_blocks(self, hidden_states, encoder_hidden_states, *args, **kwargs):
        for block in self.transformer_blocks:
            hidden_states, encoder_hidden_states = block(hidden_states, encoder_hidden_states, *args, **kwargs)
        for block in self.single_transformer_blocks:
            hidden_states, encoder_hidden_states = block(hidden_states, encoder_hidden_states, *args, **kwargs)
        return hidden_states, encoder_hidden_states

    transformer.call_transformer_blocks = call_transformer_blocks.__get__(transformer)
    transformer._is_parallelized = True
    return transformer


def parallelize_pipe(pipe, *, shallow_patch: bool = False, **kwargs):
    patch_pipe_call_for_shared_seed(pipe)
    if not shallow_patch:
        parallelize_transformer(pipe.transformer, **kwargs)
    return pipe
