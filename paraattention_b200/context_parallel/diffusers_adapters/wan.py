"""Context parallelism for Wan-shaped transformers
(src/para_attn/context_parallel/diffusers_adapters/wan.py:17-168).

The forward is re-stated from the attributes the reference uses: ``config.patch_size``,
``rope``, ``patch_embedding``, ``condition_embedder``, ``blocks``, ``scale_shift_table``,
``norm_out``, ``proj_out``. Video tokens and their rotary table are sharded along the
sequence; the text states are sharded over the batch only, so every rank's cross-attention
keys are the full prompt (replicated keys leave softmax attention unchanged).
"""
import functools
from typing import Any, Dict, Optional, Tuple

import torch

from ... import primitives as DP
from ...para_attn_interface import UnifiedAttnMode
from ._common import make_output, meshes, patch_pipe_call_for_shared_seed


def _token_grid(video: torch.Tensor, patch: Tuple[int, int, int]) -> Tuple[int, int, int]:
    """(frames, rows, columns) of the token grid a [B, C, F, H, W] latent is patchified into."""
    return tuple(extent // step for extent, step in zip(video.shape[2:], patch))


def _tokens_to_video(tokens: torch.Tensor, batch: int, grid: Tuple[int, int, int], patch: Tuple[int, int, int]):
    """[B, tokens, pt*ph*pw*C] -> [B, C, F, H, W]: every token carries one patch of every channel."""
    (gf, gh, gw), (pt, ph, pw) = grid, patch
    x = tokens.reshape(batch, gf, gh, gw, pt, ph, pw, -1)
    x = x.permute(0, 7, 1, 4, 2, 5, 3, 6)          # B, C, (gf, pt), (gh, ph), (gw, pw)
    return x.flatten(6, 7).flatten(4, 5).flatten(2, 3)


def parallelize_transformer(transformer, *, mesh=None):
    if getattr(transformer, "_is_parallelized", False):
        return transformer

    mesh, batch_mesh, seq_mesh = meshes(transformer, mesh)
    attn_mode = UnifiedAttnMode(mesh)

    def of_my_batch(x):
        return DP.get_assigned_chunk(x, dim=0, group=batch_mesh)

    def of_my_sequence(x):
        return DP.get_assigned_chunk(x, dim=-2, group=seq_mesh)

    @functools.wraps(transformer.__class__.forward)
    def new_forward(self, hidden_states: torch.Tensor, timestep: torch.LongTensor, encoder_hidden_states: torch.Tensor,
                    encoder_hidden_states_image: Optional[torch.Tensor] = None, return_dict: bool = True,
                    attention_kwargs: Optional[Dict[str, Any]] = None, **kwargs):
        batch = hidden_states.shape[0]
        patch = tuple(self.config.patch_size)
        grid = _token_grid(hidden_states, patch)

        # embeddings on the full tensors, exactly as the unsharded model computes them
        rotary_emb = self.rope(hidden_states)
        tokens = self.patch_embedding(hidden_states).flatten(2).transpose(1, 2)
        temb, timestep_proj, text, image_text = self.condition_embedder(
            timestep, encoder_hidden_states, encoder_hidden_states_image)
        timestep_proj = timestep_proj.unflatten(1, (6, -1))
        if image_text is not None:
            text = torch.concat([image_text, text], dim=1)

        # this rank's share: batch entries for everything, plus a sequence shard of the video
        # tokens and of the rotary table (which is shared by the batch)
        temb, timestep_proj, text = of_my_batch(temb), of_my_batch(timestep_proj), of_my_batch(text)
        tokens = of_my_sequence(of_my_batch(tokens))
        rotary_emb = of_my_sequence(rotary_emb)

        with attn_mode:
            tokens = self.call_transformer_blocks(tokens, text, timestep_proj, rotary_emb)

        shift, scale = (self.scale_shift_table + temb.unsqueeze(1)).chunk(2, dim=1)
        tokens = self.proj_out((self.norm_out(tokens.float()) * (1 + scale) + shift).type_as(tokens))

        tokens = DP.get_complete_tensor(tokens, dim=-2, group=seq_mesh)
        tokens = DP.get_complete_tensor(tokens, dim=0, group=batch_mesh)
        video = _tokens_to_video(tokens, batch, grid, patch)
        return make_output(getattr(self, "output_class", None), video, return_dict)

    transformer.forward = new_forward.__get__(transformer)

    def call_transformer_blocks(self, hidden_states, encoder_hidden_states, *args, **kwargs):
        # a hook point of its own: the cache adapter replaces `blocks` and expects this loop
        for block in self.blocks:
            hidden_states = block(hidden_states, encoder_hidden_states, *args, **kwargs)
        return hidden_states

    transformer.call_transformer_blocks = call_transformer_blocks.__get__(transformer)
    transformer._is_parallelized = True
    return transformer


def parallelize_pipe(pipe, *, shallow_patch: bool = False, **kwargs):
    """Patch the pipeline's call (shared seed) and, unless ``shallow_patch``, its transformer."""
    patch_pipe_call_for_shared_seed(pipe)
    if shallow_patch:
        return pipe
    parallelize_transformer(pipe.transformer, **kwargs)
    return pipe
