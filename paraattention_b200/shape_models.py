"""Shape-only diffusion transformers: random-weight stand-ins with the layer shapes, call
signatures and attribute names that the context-parallel and cache adapters touch on the
FLUX, Wan and HunyuanVideo transformers of diffusers. They exist because neither diffusers nor
any model weights are available offline; benchmarks and tests drive the adapters with them.
They are workloads, not reimplementations: normalisation and embedding details are kept only
as far as they decide tensor shapes and the number of attention calls per forward.

Every attention goes through ``F.scaled_dot_product_attention`` on ``[B, H, S, 128]`` views of
BSHD memory, which is what the attention modes intercept.
"""
from __future__ import annotations

import math
import types
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

HEAD_DIM = 128


class ShapeModelOutput:
    """Minimal stand-in for diffusers' Transformer2DModelOutput: ``.sample`` and ``[0]``."""

    def __init__(self, sample, *rest):
        self.sample = sample
        self._rest = rest

    def __getitem__(self, i):
        return ((self.sample,) + tuple(self._rest))[i]


def _split_heads(x: torch.Tensor) -> torch.Tensor:
    return x.unflatten(-1, (-1, HEAD_DIM)).transpose(1, 2)  # [B, S, H*D] -> [B, H, S, D] view


def _merge_heads(x: torch.Tensor) -> torch.Tensor:
    return x.transpose(1, 2).flatten(2)


def _rms(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, H, S, D]; cos, sin: [S, D] (broadcast over batch and heads)."""
    x1, x2 = x[..., ::2], x[..., 1::2]
    rot = torch.stack((-x2, x1), dim=-1).flatten(-2)
    return (x.float() * cos + rot.float() * sin).to(x.dtype)


def _joint_qkv(streams, rotary, rotary_rows=None):
    """q, k, v of one attention call from the projection outputs of its streams.

    ``streams``: list of ``(q, k, v, q_weight, k_weight)`` in sequence order, q/k/v [B, S_i, H*D]
    projection outputs (any row stride), weights [D] or None. ``rotary``: (cos, sin) or None;
    ``rotary_rows = (first, count)`` limits the rotation to those rows of the joint sequence,
    table row 0 belonging to joint row ``first`` (default: all rows). Returns [B, H, sum S_i, D] views.

    On CUDA bf16/f16 tensors each stream is one launch of the fused kernel (three when only a
    part of it rotates), which normalises, rotates and writes into the joint buffers
    (``config.attention.fuse_qkv_prepare``); otherwise the same arithmetic runs as the chain of
    tensor operations below."""
    from . import config

    q0 = streams[0][0]
    total = sum(st[0].shape[1] for st in streams)
    first, count = (0, total) if rotary_rows is None else rotary_rows
    if config.attention.fuse_qkv_prepare and q0.device.type == "cuda" and q0.dtype in (torch.bfloat16, torch.float16):
        from . import ops

        B, H = q0.shape[0], q0.shape[2] // HEAD_DIM
        bufs = tuple(torch.empty((B, total, H, HEAD_DIM), dtype=q0.dtype, device=q0.device).transpose(1, 2)
                     for _ in range(3))
        off = 0
        for q, k, v, wq, wk in streams:
            rows = q.shape[1]
            lo, hi = max(off, first), min(off + rows, first + count)  # joint rows of this stream that rotate
            if rotary is None or hi <= lo:
                segments = [(0, rows, False)]
            else:
                segments = [(0, lo - off, False), (lo - off, hi - off, True), (hi - off, rows, False)]
            for a, b, rotate in segments:
                if b <= a:
                    continue
                joint_row = off + a
                table_row = joint_row - first if rotate else joint_row
                # destination views cut so that their row index equals the table row index
                dst = tuple(buf[:, :, joint_row - table_row:] for buf in bufs)
                ops.qkv_prepare(_split_heads(q[:, a:b]), _split_heads(k[:, a:b]), _split_heads(v[:, a:b]), wq, wk,
                                rotary if rotate else None, out=dst, row_offset=table_row)
            off += rows
        return bufs
    qs, ks, vs = [], [], []
    for q, k, v, wq, wk in streams:
        q, k, v = _split_heads(q), _split_heads(k), _split_heads(v)
        qs.append(_rms(q, wq) if wq is not None else q)
        ks.append(_rms(k, wk) if wk is not None else k)
        vs.append(v)
    q, k, v = (torch.cat(t, dim=2) if len(t) > 1 else t[0] for t in (qs, ks, vs))
    if rotary is not None:
        cos, sin = rotary
        if first == 0 and count == total:
            q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        else:
            sl = slice(first, first + count)
            q = torch.cat([q[:, :, :first], _rope(q[:, :, sl], cos, sin), q[:, :, first + count:]], dim=2)
            k = torch.cat([k[:, :, :first], _rope(k[:, :, sl], cos, sin), k[:, :, first + count:]], dim=2)
    return q, k, v


def _rope_table(positions: torch.Tensor, axes_dim=(16, 56, 56), theta: float = 10000.0):
    """positions: [S, 3] -> (cos, sin) of shape [S, sum(axes_dim)] with pairwise-repeated frequencies."""
    outs = []
    for a, d in enumerate(axes_dim):
        freqs = 1.0 / (theta ** (torch.arange(0, d, 2, device=positions.device, dtype=torch.float32) / d))
        ang = positions[:, a].float()[:, None] * freqs[None, :]
        outs.append(ang.repeat_interleave(2, dim=-1))
    ang = torch.cat(outs, dim=-1)
    return ang.cos(), ang.sin()


def _timestep_embedding(t: torch.Tensor, dim: int = 256) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    args = t.float().reshape(-1, 1) * freqs[None]
    return torch.cat([args.cos(), args.sin()], dim=-1)


class _Modulation(nn.Module):
    """adaLN: silu(temb) -> n chunks of [B, 1, dim]."""

    def __init__(self, dim: int, n: int):
        super().__init__()
        self.n = n
        self.linear = nn.Linear(dim, n * dim)

    def forward(self, temb):
        return self.linear(F.silu(temb)).unsqueeze(1).chunk(self.n, dim=-1)


class _FeedForward(nn.Module):
    def __init__(self, dim: int, inner: int):
        super().__init__()
        self.up = nn.Linear(dim, inner)
        self.down = nn.Linear(inner, dim)

    def forward(self, x):
        return self.down(F.gelu(self.up(x), approximate="tanh"))


class _TimeTextEmbed(nn.Module):
    def __init__(self, dim: int, pooled_dim: int, with_guidance: bool):
        super().__init__()
        self.time = nn.Sequential(nn.Linear(256, dim), nn.SiLU(), nn.Linear(dim, dim))
        self.guidance = nn.Sequential(nn.Linear(256, dim), nn.SiLU(), nn.Linear(dim, dim)) if with_guidance else None
        self.text = nn.Sequential(nn.Linear(pooled_dim, dim), nn.SiLU(), nn.Linear(dim, dim))

    def forward(self, timestep, guidance, pooled_projections):
        dtype = pooled_projections.dtype
        emb = self.time(_timestep_embedding(timestep).to(dtype))
        if self.guidance is not None and guidance is not None:
            emb = emb + self.guidance(_timestep_embedding(guidance).to(dtype))
        return emb + self.text(pooled_projections)


def _norm(x: torch.Tensor) -> torch.Tensor:
    return F.layer_norm(x.float(), x.shape[-1:]).to(x.dtype)


class _DeviceMixin:
    @property
    def device(self):
        return next(self.parameters()).device

    @property
    def dtype(self):
        return next(self.parameters()).dtype


def _attention(q, k, v):
    return _merge_heads(F.scaled_dot_product_attention(q, k, v))


# ==============================================================================================
# FLUX-shaped MMDiT: 19 dual-stream + 38 single-stream blocks, hidden 3072 = 24 heads x 128
# ==============================================================================================
class _JointStream(nn.Module):
    """One stream (image or text) of a dual-stream block: modulation, qkv, per-head q/k norm."""

    def __init__(self, dim: int, mlp_ratio: float):
        super().__init__()
        self.mod = _Modulation(dim, 6)
        self.qkv = nn.Linear(dim, 3 * dim)
        self.q_norm = nn.Parameter(torch.ones(HEAD_DIM))
        self.k_norm = nn.Parameter(torch.ones(HEAD_DIM))
        self.out = nn.Linear(dim, dim)
        self.ff = _FeedForward(dim, int(dim * mlp_ratio))

    def qkv_heads(self, x, temb):
        shift, scale, gate, shift2, scale2, gate2 = self.mod(temb)
        q, k, v = self.qkv(_norm(x) * (1 + scale) + shift).chunk(3, dim=-1)
        q, k, v = _split_heads(q), _split_heads(k), _split_heads(v)
        return _rms(q, self.q_norm), _rms(k, self.k_norm), v, (gate, shift2, scale2, gate2)

    def qkv_stream(self, x, temb):
        """The raw projections and norm weights as a stream of ``_joint_qkv``, plus the modulation."""
        shift, scale, gate, shift2, scale2, gate2 = self.mod(temb)
        q, k, v = self.qkv(_norm(x) * (1 + scale) + shift).chunk(3, dim=-1)
        return (q, k, v, self.q_norm, self.k_norm), (gate, shift2, scale2, gate2)

    def finish(self, x, attn, mods):
        gate, shift2, scale2, gate2 = mods
        x = x + gate * self.out(attn)
        return x + gate2 * self.ff(_norm(x) * (1 + scale2) + shift2)


class FluxDualStreamBlock(nn.Module):
    def __init__(self, dim: int, mlp_ratio: float = 4.0):
        super().__init__()
        self.img = _JointStream(dim, mlp_ratio)
        self.txt = _JointStream(dim, mlp_ratio)

    def forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb=None, **kwargs):
        img, mi = self.img.qkv_stream(hidden_states, temb)
        txt, mt = self.txt.qkv_stream(encoder_hidden_states, temb)
        attn = _attention(*_joint_qkv([txt, img], image_rotary_emb))
        n_txt = encoder_hidden_states.shape[1]
        encoder_hidden_states = self.txt.finish(encoder_hidden_states, attn[:, :n_txt], mt)
        hidden_states = self.img.finish(hidden_states, attn[:, n_txt:], mi)
        return encoder_hidden_states, hidden_states


class FluxSingleStreamBlock(nn.Module):
    def __init__(self, dim: int, mlp_ratio: float = 4.0):
        super().__init__()
        self.mod = _Modulation(dim, 3)
        self.qkv_mlp = nn.Linear(dim, 3 * dim + int(dim * mlp_ratio))
        self.q_norm = nn.Parameter(torch.ones(HEAD_DIM))
        self.k_norm = nn.Parameter(torch.ones(HEAD_DIM))
        self.out = nn.Linear(dim + int(dim * mlp_ratio), dim)
        self.dim = dim

    def forward(self, hidden_states, temb, image_rotary_emb=None, **kwargs):
        shift, scale, gate = self.mod(temb)
        qkv, mlp = self.qkv_mlp(_norm(hidden_states) * (1 + scale) + shift).split([3 * self.dim, self.qkv_mlp.out_features - 3 * self.dim], dim=-1)
        q, k, v = qkv.chunk(3, dim=-1)
        attn = _attention(*_joint_qkv([(q, k, v, self.q_norm, self.k_norm)], image_rotary_emb))
        return hidden_states + gate * self.out(torch.cat([attn, F.gelu(mlp, approximate="tanh")], dim=-1))


class FluxShapedTransformer2DModel(nn.Module, _DeviceMixin):
    """FLUX.1-dev shapes by default: joint attention over 512 text + 4096 image tokens."""

    def __init__(self, dim: int = 3072, num_layers: int = 19, num_single_layers: int = 38, in_channels: int = 64,
                 joint_attention_dim: int = 4096, pooled_projection_dim: int = 768, mlp_ratio: float = 4.0,
                 axes_dims_rope=(16, 56, 56), guidance_embeds: bool = True):
        super().__init__()
        assert dim % HEAD_DIM == 0
        self.config = types.SimpleNamespace(num_attention_heads=dim // HEAD_DIM, attention_head_dim=HEAD_DIM,
                                            in_channels=in_channels, joint_attention_dim=joint_attention_dim,
                                            axes_dims_rope=tuple(axes_dims_rope))
        self.x_embedder = nn.Linear(in_channels, dim)
        self.context_embedder = nn.Linear(joint_attention_dim, dim)
        self.time_text_embed = _TimeTextEmbed(dim, pooled_projection_dim, guidance_embeds)
        self.transformer_blocks = nn.ModuleList([FluxDualStreamBlock(dim, mlp_ratio) for _ in range(num_layers)])
        self.single_transformer_blocks = nn.ModuleList(
            [FluxSingleStreamBlock(dim, mlp_ratio) for _ in range(num_single_layers)])
        self.norm_out = _Modulation(dim, 2)
        self.proj_out = nn.Linear(dim, in_channels)

    def forward(self, hidden_states, encoder_hidden_states=None, pooled_projections=None, timestep=None, img_ids=None,
                txt_ids=None, guidance=None, return_dict: bool = True, **kwargs):
        hidden_states = self.x_embedder(hidden_states)
        temb = self.time_text_embed(timestep, guidance, pooled_projections)
        encoder_hidden_states = self.context_embedder(encoder_hidden_states)
        ids = torch.cat((txt_ids, img_ids), dim=0)
        image_rotary_emb = _rope_table(ids, self.config.axes_dims_rope)
        for block in self.transformer_blocks:
            encoder_hidden_states, hidden_states = block(
                hidden_states=hidden_states, encoder_hidden_states=encoder_hidden_states, temb=temb,
                image_rotary_emb=image_rotary_emb)
        n_txt = encoder_hidden_states.shape[1]
        hidden_states = torch.cat([encoder_hidden_states, hidden_states], dim=1)
        for block in self.single_transformer_blocks:
            hidden_states = block(hidden_states=hidden_states, temb=temb, image_rotary_emb=image_rotary_emb)
        hidden_states = hidden_states[:, n_txt:]
        shift, scale = self.norm_out(temb)
        output = self.proj_out(_norm(hidden_states) * (1 + scale) + shift)
        if not return_dict:
            return (output,)
        return ShapeModelOutput(output)


class FluxShapedPipeline:
    """Denoising loop around the transformer: what ``parallelize_pipe`` / ``apply_cache_on_pipe`` patch."""

    def __init__(self, transformer: FluxShapedTransformer2DModel, text_tokens: int = 512, latent_hw=(64, 64)):
        self.transformer = transformer
        self.text_tokens = text_tokens
        self.latent_hw = latent_hw

    @property
    def device(self):
        return self.transformer.device

    def __call__(self, num_inference_steps: int = 28, generator=None, prompt_seed: int = 0, output_trace=None):
        dev, dt = self.device, self.transformer.dtype
        cfg = self.transformer.config
        h, w = self.latent_hw
        g = generator if generator is not None else torch.Generator(dev).manual_seed(0)
        latents = torch.randn(1, h * w, cfg.in_channels, generator=g, device=dev).to(dt)
        pg = torch.Generator(dev).manual_seed(prompt_seed)
        enc = torch.randn(1, self.text_tokens, cfg.joint_attention_dim, generator=pg, device=dev).to(dt)
        pooled = torch.randn(1, 768, generator=pg, device=dev).to(dt)
        ys, xs = torch.meshgrid(torch.arange(h, device=dev), torch.arange(w, device=dev), indexing="ij")
        img_ids = torch.stack([torch.zeros_like(ys), ys, xs], dim=-1).reshape(-1, 3).float()
        txt_ids = torch.zeros(self.text_tokens, 3, device=dev)
        guidance = torch.full((1,), 3.5, device=dev)
        sigmas = torch.linspace(1.0, 1.0 / num_inference_steps, num_inference_steps, device=dev)
        for i in range(num_inference_steps):
            t = sigmas[i].expand(1)
            pred = self.transformer(hidden_states=latents, encoder_hidden_states=enc, pooled_projections=pooled,
                                    timestep=t * 1000, img_ids=img_ids, txt_ids=txt_ids, guidance=guidance,
                                    return_dict=False)[0]
            nxt = sigmas[i + 1] if i + 1 < num_inference_steps else torch.zeros((), device=dev)
            latents = (latents.float() + (nxt - sigmas[i]) * pred.float()).to(dt)
            if output_trace is not None:
                output_trace.append(pred)
        return latents
