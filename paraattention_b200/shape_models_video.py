"""Shape-only video diffusion transformers (Wan 2.1 14B-shaped and HunyuanVideo-shaped); see
``shape_models`` for what "shape-only" means. Attribute names and block signatures follow what
the adapters use (src/para_attn/context_parallel/diffusers_adapters/wan.py:49-104,
hunyuan_video.py:50-131 of the reference)."""
from __future__ import annotations

import types
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .shape_models import (HEAD_DIM, ShapeModelOutput, _attention, _DeviceMixin, _FeedForward, _Modulation, _norm,
                           _joint_qkv, _rms, _rope, _rope_table, _split_heads, _timestep_embedding, _TimeTextEmbed)


def _grid_positions(frames: int, height: int, width: int, device) -> torch.Tensor:
    f, h, w = torch.meshgrid(torch.arange(frames, device=device), torch.arange(height, device=device),
                             torch.arange(width, device=device), indexing="ij")
    return torch.stack([f, h, w], dim=-1).reshape(-1, 3).float()


# ==============================================================================================
# Wan 2.1 14B-shaped: dim 5120 = 40 heads x 128, 40 blocks, FFN 13824, text cross-attention
# ==============================================================================================
class _WanRope(nn.Module):
    def __init__(self, patch_size, axes_dim=(44, 42, 42)):
        super().__init__()
        self.patch_size, self.axes_dim = patch_size, axes_dim

    def forward(self, hidden_states):
        _, _, f, h, w = hidden_states.shape
        p_t, p_h, p_w = self.patch_size
        cos, sin = _rope_table(_grid_positions(f // p_t, h // p_h, w // p_w, hidden_states.device), self.axes_dim)
        return torch.cat([cos, sin], dim=-1)[None, None]  # [1, 1, N, 2*128]: sequence on dim -2


class _WanConditionEmbedder(nn.Module):
    def __init__(self, dim: int, text_dim: int):
        super().__init__()
        self.time = nn.Sequential(nn.Linear(256, dim), nn.SiLU(), nn.Linear(dim, dim))
        self.time_proj = nn.Linear(dim, 6 * dim)
        self.text = nn.Sequential(nn.Linear(text_dim, dim), nn.GELU(approximate="tanh"), nn.Linear(dim, dim))

    def forward(self, timestep, encoder_hidden_states, encoder_hidden_states_image=None):
        temb = self.time(_timestep_embedding(timestep).to(encoder_hidden_states.dtype))
        return temb, self.time_proj(F.silu(temb)), self.text(encoder_hidden_states), encoder_hidden_states_image


class WanShapedBlock(nn.Module):
    def __init__(self, dim: int, ffn_dim: int):
        super().__init__()
        self.scale_shift_table = nn.Parameter(torch.randn(1, 6, dim) / dim ** 0.5)
        self.qkv = nn.Linear(dim, 3 * dim)
        self.q_norm, self.k_norm = nn.Parameter(torch.ones(HEAD_DIM)), nn.Parameter(torch.ones(HEAD_DIM))
        self.out = nn.Linear(dim, dim)
        self.cross_q = nn.Linear(dim, dim)
        self.cross_kv = nn.Linear(dim, 2 * dim)
        self.cross_out = nn.Linear(dim, dim)
        self.ffn = _FeedForward(dim, ffn_dim)

    def forward(self, hidden_states, encoder_hidden_states, temb, rotary_emb):
        shift, scale, gate, c_shift, c_scale, c_gate = (self.scale_shift_table + temb.float()).to(
            hidden_states.dtype).chunk(6, dim=1)
        cos, sin = rotary_emb[0, 0].chunk(2, dim=-1)
        q, k, v = self.qkv(_norm(hidden_states) * (1 + scale) + shift).chunk(3, dim=-1)
        q, k, v = _joint_qkv([(q, k, v, self.q_norm, self.k_norm)], (cos.contiguous(), sin.contiguous()))
        hidden_states = hidden_states + gate * self.out(_attention(q, k, v))
        # cross-attention to the prompt
        cq = _split_heads(self.cross_q(_norm(hidden_states)))
        ck, cv = self.cross_kv(encoder_hidden_states).chunk(2, dim=-1)
        hidden_states = hidden_states + self.cross_out(_attention(cq, _split_heads(ck), _split_heads(cv)))
        return hidden_states + c_gate * self.ffn(_norm(hidden_states) * (1 + c_scale) + c_shift)


class WanShapedTransformer3DModel(nn.Module, _DeviceMixin):
    """Defaults: 480x832, 81 frames -> latent 16 x 21 x 60 x 104, patch (1,2,2) -> 32760 tokens."""

    def __init__(self, dim: int = 5120, num_layers: int = 40, ffn_dim: int = 13824, in_channels: int = 16,
                 text_dim: int = 4096, patch_size=(1, 2, 2)):
        super().__init__()
        assert dim % HEAD_DIM == 0
        self.config = types.SimpleNamespace(patch_size=tuple(patch_size), num_attention_heads=dim // HEAD_DIM,
                                            in_channels=in_channels, text_dim=text_dim)
        self.rope = _WanRope(tuple(patch_size))
        self.patch_embedding = nn.Conv3d(in_channels, dim, kernel_size=patch_size, stride=patch_size)
        self.condition_embedder = _WanConditionEmbedder(dim, text_dim)
        self.blocks = nn.ModuleList([WanShapedBlock(dim, ffn_dim) for _ in range(num_layers)])
        self.scale_shift_table = nn.Parameter(torch.randn(1, 2, dim) / dim ** 0.5)
        self.norm_out = lambda x: F.layer_norm(x, x.shape[-1:])
        self.proj_out = nn.Linear(dim, in_channels * patch_size[0] * patch_size[1] * patch_size[2])
        self.gradient_checkpointing = False

    def forward(self, hidden_states, timestep, encoder_hidden_states, encoder_hidden_states_image=None,
                return_dict: bool = True, attention_kwargs=None, **kwargs):
        batch_size, _, num_frames, height, width = hidden_states.shape
        p_t, p_h, p_w = self.config.patch_size
        ppf, pph, ppw = num_frames // p_t, height // p_h, width // p_w
        rotary_emb = self.rope(hidden_states)
        hidden_states = self.patch_embedding(hidden_states).flatten(2).transpose(1, 2)
        temb, timestep_proj, encoder_hidden_states, _ = self.condition_embedder(
            timestep, encoder_hidden_states, encoder_hidden_states_image)
        timestep_proj = timestep_proj.unflatten(1, (6, -1))
        for block in self.blocks:
            hidden_states = block(hidden_states, encoder_hidden_states, timestep_proj, rotary_emb)
        shift, scale = (self.scale_shift_table + temb.unsqueeze(1)).chunk(2, dim=1)
        hidden_states = (self.norm_out(hidden_states.float()) * (1 + scale) + shift).type_as(hidden_states)
        hidden_states = self.proj_out(hidden_states)
        hidden_states = hidden_states.reshape(batch_size, ppf, pph, ppw, p_t, p_h, p_w, -1)
        output = hidden_states.permute(0, 7, 1, 4, 2, 5, 3, 6).flatten(6, 7).flatten(4, 5).flatten(2, 3)
        if not return_dict:
            return (output,)
        return ShapeModelOutput(output)
