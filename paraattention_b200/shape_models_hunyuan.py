"""Shape-only HunyuanVideo-shaped transformer (see ``shape_models``): hidden 3072 = 24 heads x
128, 20 dual-stream + 40 single-stream blocks, joint attention over video + text tokens. Block
signature ``block(hidden_states, encoder_hidden_states, temb, attention_mask,
image_rotary_emb) -> (hidden_states, encoder_hidden_states)`` for both block kinds, as the
reference's adapters assume (src/para_attn/context_parallel/diffusers_adapters/hunyuan_video.py:162-197)."""
from __future__ import annotations

import types

import torch
import torch.nn as nn
import torch.nn.functional as F

from .shape_models import (HEAD_DIM, ShapeModelOutput, _attention, _DeviceMixin, _Modulation, _norm, _rms, _rope,
                           _joint_qkv, _rope_table, _split_heads, _TimeTextEmbed, _JointStream)
from .shape_models_video import _grid_positions


class _HunyuanRope(nn.Module):
    def __init__(self, patch_size: int, patch_size_t: int, axes_dim=(16, 56, 56)):
        super().__init__()
        self.p, self.p_t, self.axes_dim = patch_size, patch_size_t, axes_dim

    def forward(self, hidden_states):
        _, _, f, h, w = hidden_states.shape
        return _rope_table(_grid_positions(f // self.p_t, h // self.p, w // self.p, hidden_states.device),
                           self.axes_dim)  # (cos, sin), each [N, 128]


class _PatchEmbed(nn.Module):
    def __init__(self, in_channels, dim, patch_size, patch_size_t):
        super().__init__()
        k = (patch_size_t, patch_size, patch_size)
        self.proj = nn.Conv3d(in_channels, dim, kernel_size=k, stride=k)

    def forward(self, x):
        return self.proj(x).flatten(2).transpose(1, 2)


class _ContextEmbedder(nn.Module):
    def __init__(self, text_dim, dim):
        super().__init__()
        self.proj = nn.Sequential(nn.Linear(text_dim, dim), nn.SiLU(), nn.Linear(dim, dim))

    def forward(self, encoder_hidden_states, timestep, attention_mask=None):
        return self.proj(encoder_hidden_states)


class HunyuanDualStreamBlock(nn.Module):
    def __init__(self, dim: int, mlp_ratio: float = 4.0):
        super().__init__()
        self.img = _JointStream(dim, mlp_ratio)
        self.txt = _JointStream(dim, mlp_ratio)

    def forward(self, hidden_states, encoder_hidden_states, temb, attention_mask=None, image_rotary_emb=None):
        img, mi = self.img.qkv_stream(hidden_states, temb)
        txt, mt = self.txt.qkv_stream(encoder_hidden_states, temb)
        n_img = hidden_states.shape[1]
        # rotary embedding on the video tokens (the first n_img of the joint sequence) only
        q, k, v = _joint_qkv([img, txt], image_rotary_emb, rotary_rows=(0, n_img))
        attn = F.scaled_dot_product_attention(q, k, v, attn_mask=attention_mask).transpose(1, 2).flatten(2)
        hidden_states = self.img.finish(hidden_states, attn[:, :n_img], mi)
        encoder_hidden_states = self.txt.finish(encoder_hidden_states, attn[:, n_img:], mt)
        return hidden_states, encoder_hidden_states


class HunyuanSingleStreamBlock(nn.Module):
    def __init__(self, dim: int, mlp_ratio: float = 4.0):
        super().__init__()
        self.dim, self.mlp = dim, int(dim * mlp_ratio)
        self.mod = _Modulation(dim, 3)
        self.qkv_mlp = nn.Linear(dim, 3 * dim + self.mlp)
        self.q_norm, self.k_norm = nn.Parameter(torch.ones(HEAD_DIM)), nn.Parameter(torch.ones(HEAD_DIM))
        self.out = nn.Linear(dim + self.mlp, dim)

    def forward(self, hidden_states, encoder_hidden_states, temb, attention_mask=None, image_rotary_emb=None):
        n_img = hidden_states.shape[1]
        x = torch.cat([hidden_states, encoder_hidden_states], dim=1)
        shift, scale, gate = self.mod(temb)
        qkv, mlp = self.qkv_mlp(_norm(x) * (1 + scale) + shift).split([3 * self.dim, self.mlp], dim=-1)
        q, k, v = qkv.chunk(3, dim=-1)
        q, k, v = _joint_qkv([(q, k, v, self.q_norm, self.k_norm)], image_rotary_emb, rotary_rows=(0, n_img))
        attn = F.scaled_dot_product_attention(q, k, v, attn_mask=attention_mask).transpose(1, 2).flatten(2)
        x = x + gate * self.out(torch.cat([attn, F.gelu(mlp, approximate="tanh")], dim=-1))
        return x[:, :n_img], x[:, n_img:]


class _AdaNormOut(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.mod = _Modulation(dim, 2)

    def forward(self, x, temb):
        shift, scale = self.mod(temb)
        return _norm(x) * (1 + scale) + shift


class HunyuanVideoShapedTransformer3DModel(nn.Module, _DeviceMixin):
    """Defaults: 720x1280, 129 frames -> latent 16 x 33 x 90 x 160, patch (1,2,2) -> 118800 tokens."""

    def __init__(self, dim: int = 3072, num_layers: int = 20, num_single_layers: int = 40, in_channels: int = 16,
                 text_dim: int = 4096, pooled_projection_dim: int = 768, patch_size: int = 2, patch_size_t: int = 1,
                 mlp_ratio: float = 4.0):
        super().__init__()
        assert dim % HEAD_DIM == 0
        self.config = types.SimpleNamespace(patch_size=patch_size, patch_size_t=patch_size_t, in_channels=in_channels,
                                            num_attention_heads=dim // HEAD_DIM, text_embed_dim=text_dim)
        self.rope = _HunyuanRope(patch_size, patch_size_t)
        self.time_text_embed = _TimeTextEmbed(dim, pooled_projection_dim, True)
        self.x_embedder = _PatchEmbed(in_channels, dim, patch_size, patch_size_t)
        self.context_embedder = _ContextEmbedder(text_dim, dim)
        self.transformer_blocks = nn.ModuleList([HunyuanDualStreamBlock(dim, mlp_ratio) for _ in range(num_layers)])
        self.single_transformer_blocks = nn.ModuleList(
            [HunyuanSingleStreamBlock(dim, mlp_ratio) for _ in range(num_single_layers)])
        self.norm_out = _AdaNormOut(dim)
        self.proj_out = nn.Linear(dim, in_channels * patch_size_t * patch_size * patch_size)
        self.gradient_checkpointing = False

    def forward(self, hidden_states, timestep, encoder_hidden_states, encoder_attention_mask, pooled_projections,
                guidance=None, attention_kwargs=None, return_dict: bool = True, **kwargs):
        batch_size, _, num_frames, height, width = hidden_states.shape
        p, p_t = self.config.patch_size, self.config.patch_size_t
        ppf, pph, ppw = num_frames // p_t, height // p, width // p
        image_rotary_emb = self.rope(hidden_states)
        temb = self.time_text_embed(timestep, guidance, pooled_projections)
        hidden_states = self.x_embedder(hidden_states)
        encoder_hidden_states = self.context_embedder(encoder_hidden_states, timestep, encoder_attention_mask)
        # key-padding mask over [video tokens, prompt tokens]; None when the prompt has no padding
        attention_mask = None
        if encoder_attention_mask is not None and not bool(encoder_attention_mask.to(torch.bool).all()):
            video = torch.ones(batch_size, hidden_states.shape[1], dtype=torch.bool, device=hidden_states.device)
            attention_mask = torch.cat([video, encoder_attention_mask.to(torch.bool)], dim=1)[:, None, None, :]
        for block in self.transformer_blocks:
            hidden_states, encoder_hidden_states = block(hidden_states, encoder_hidden_states, temb, attention_mask,
                                                         image_rotary_emb)
        for block in self.single_transformer_blocks:
            hidden_states, encoder_hidden_states = block(hidden_states, encoder_hidden_states, temb, attention_mask,
                                                         image_rotary_emb)
        hidden_states = self.proj_out(self.norm_out(hidden_states, temb))
        hidden_states = hidden_states.reshape(batch_size, ppf, pph, ppw, -1, p_t, p, p)
        hidden_states = hidden_states.permute(0, 4, 1, 5, 2, 6, 3, 7).flatten(6, 7).flatten(4, 5).flatten(2, 3)
        if not return_dict:
            return (hidden_states,)
        return ShapeModelOutput(hidden_states)
