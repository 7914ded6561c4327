"""Text token refiner (``teletron/models/hunyuanvideo/layers.py:37-206``).

Two pre-LN transformer blocks over the (<= 256) LLaMA text tokens, gated by a
timestep + masked-mean-pooled-text embedding.  Sub-module names reproduce the
diffusers layout (``attn.to_q``, ``attn.to_out.0``, ``ff.net.0.proj``, ``ff.net.2``) so
the identical-weight list of the checkpoint converter applies unchanged.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn
import torch.nn.functional as F

from .embeddings import CombinedTimestepTextProjEmbeddings


class _RefinerAttention(nn.Module):
    def __init__(self, dim: int, heads: int, head_dim: int, bias: bool = True):
        super().__init__()
        self.heads, self.head_dim = heads, head_dim
        inner = heads * head_dim
        self.to_q = nn.Linear(dim, inner, bias=bias)
        self.to_k = nn.Linear(dim, inner, bias=bias)
        self.to_v = nn.Linear(dim, inner, bias=bias)
        self.to_out = nn.ModuleList([nn.Linear(inner, dim, bias=True), nn.Identity()])

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor]) -> torch.Tensor:
        B, T, _ = x.shape
        q = self.to_q(x).view(B, T, self.heads, self.head_dim).transpose(1, 2)
        k = self.to_k(x).view(B, T, self.heads, self.head_dim).transpose(1, 2)
        v = self.to_v(x).view(B, T, self.heads, self.head_dim).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        return self.to_out[0](o.transpose(1, 2).reshape(B, T, -1))


class _LinearSiLU(nn.Module):
    def __init__(self, dim: int, inner: int):
        super().__init__()
        self.proj = nn.Linear(dim, inner)

    def forward(self, x):
        return F.silu(self.proj(x))


class _FeedForward(nn.Module):
    """``net.0.proj`` Linear + SiLU, dropout (identity at rate 0), ``net.2`` Linear."""

    def __init__(self, dim: int, mult: float):
        super().__init__()
        inner = int(dim * mult)
        self.net = nn.ModuleList([_LinearSiLU(dim, inner), nn.Identity(), nn.Linear(inner, dim)])

    def forward(self, x):
        return self.net[2](self.net[0](x))


class HunyuanVideoAdaNorm(nn.Module):
    def __init__(self, in_features: int, out_features: Optional[int] = None):
        super().__init__()
        self.linear = nn.Linear(in_features, out_features or 2 * in_features)

    def forward(self, temb):
        gate_msa, gate_mlp = self.linear(F.silu(temb)).chunk(2, dim=1)
        return gate_msa.unsqueeze(1), gate_mlp.unsqueeze(1)


class HunyuanVideoIndividualTokenRefinerBlock(nn.Module):
    def __init__(self, heads: int, head_dim: int, mlp_width_ratio: float = 4.0, attention_bias: bool = True):
        super().__init__()
        dim = heads * head_dim
        self.norm1 = nn.LayerNorm(dim, elementwise_affine=True, eps=1e-6)
        self.attn = _RefinerAttention(dim, heads, head_dim, attention_bias)
        self.norm2 = nn.LayerNorm(dim, elementwise_affine=True, eps=1e-6)
        self.ff = _FeedForward(dim, mlp_width_ratio)
        self.norm_out = HunyuanVideoAdaNorm(dim, 2 * dim)

    def forward(self, x, temb, mask=None):
        gate_msa, gate_mlp = self.norm_out(temb)
        x = x + self.attn(self.norm1(x), mask) * gate_msa
        return x + self.ff(self.norm2(x)) * gate_mlp


class HunyuanVideoIndividualTokenRefiner(nn.Module):
    def __init__(self, heads: int, head_dim: int, num_layers: int, mlp_width_ratio: float = 4.0,
                 attention_bias: bool = True):
        super().__init__()
        self.refiner_blocks = nn.ModuleList(
            [HunyuanVideoIndividualTokenRefinerBlock(heads, head_dim, mlp_width_ratio, attention_bias)
             for _ in range(num_layers)])

    def forward(self, x, temb, attention_mask=None):
        mask = None
        if attention_mask is not None:
            m = attention_mask.to(x.device).bool()                      # [B, T]
            mask = m[:, None, None, :] & m[:, None, :, None]             # pairwise validity
            mask = mask.clone()
            mask[:, :, :, 0] = True                                      # every row keeps one valid key
        for blk in self.refiner_blocks:
            x = blk(x, temb, mask)
        return x


class HunyuanVideoTokenRefiner(nn.Module):
    def __init__(self, in_channels: int, heads: int, head_dim: int, num_layers: int, mlp_ratio: float = 4.0,
                 attention_bias: bool = True):
        super().__init__()
        dim = heads * head_dim
        self.time_text_embed = CombinedTimestepTextProjEmbeddings(dim, in_channels)
        self.proj_in = nn.Linear(in_channels, dim, bias=True)
        self.token_refiner = HunyuanVideoIndividualTokenRefiner(heads, head_dim, num_layers, mlp_ratio, attention_bias)

    def forward(self, hidden_states, timestep, attention_mask=None):
        if attention_mask is None:
            pooled = hidden_states.mean(dim=1)
        else:
            mf = attention_mask.to(hidden_states.device).float().unsqueeze(-1)
            pooled = ((hidden_states.float() * mf).sum(dim=1) / mf.sum(dim=1).clamp_min(1.0)).to(hidden_states.dtype)
        temb = self.time_text_embed(timestep, pooled)
        return self.token_refiner(self.proj_in(hidden_states), temb, attention_mask)
