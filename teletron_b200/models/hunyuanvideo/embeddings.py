"""Condition embedders, patch embedding and the 3-axis rotary table.

The reference imports these from ``diffusers`` (``teletron/models/hunyuanvideo/layers.py:6-12``);
they are restated here with the same parameter names so converted checkpoints load
unchanged (``convert_hunyuanvideo.py:126-189`` lists the names).
"""

from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
from torch import nn
import torch.nn.functional as F


def sinusoidal_timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: float = 10000.0) -> torch.Tensor:
    """``[cos | sin]`` sinusoid (``flip_sin_to_cos=True``, ``downscale_freq_shift=0``)."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


class TimestepEmbedding(nn.Module):
    def __init__(self, in_dim: int, dim: int):
        super().__init__()
        self.linear_1 = nn.Linear(in_dim, dim)
        self.linear_2 = nn.Linear(dim, dim)

    def forward(self, x):
        return self.linear_2(F.silu(self.linear_1(x)))


class TextProjection(nn.Module):
    """``linear_1 -> SiLU -> linear_2`` on the pooled text vector."""

    def __init__(self, in_dim: int, dim: int):
        super().__init__()
        self.linear_1 = nn.Linear(in_dim, dim)
        self.linear_2 = nn.Linear(dim, dim)

    def forward(self, x):
        return self.linear_2(F.silu(self.linear_1(x)))


class CombinedTimestepGuidanceTextProjEmbeddings(nn.Module):
    """timestep + guidance + pooled-text embedding -> ``temb [B, dim]`` (``model.py:287``)."""

    def __init__(self, embedding_dim: int, pooled_projection_dim: int, guidance: bool = True):
        super().__init__()
        self.timestep_embedder = TimestepEmbedding(256, embedding_dim)
        self.guidance_embedder = TimestepEmbedding(256, embedding_dim) if guidance else None
        self.text_embedder = TextProjection(pooled_projection_dim, embedding_dim)

    def forward(self, timestep, guidance, pooled_projection):
        dtype = pooled_projection.dtype
        emb = self.timestep_embedder(sinusoidal_timestep_embedding(timestep).to(dtype))
        if self.guidance_embedder is not None and guidance is not None:
            emb = emb + self.guidance_embedder(sinusoidal_timestep_embedding(guidance).to(dtype))
        return emb + self.text_embedder(pooled_projection)


class CombinedTimestepTextProjEmbeddings(nn.Module):
    def __init__(self, embedding_dim: int, pooled_projection_dim: int):
        super().__init__()
        self.timestep_embedder = TimestepEmbedding(256, embedding_dim)
        self.text_embedder = TextProjection(pooled_projection_dim, embedding_dim)

    def forward(self, timestep, pooled_projection):
        dtype = pooled_projection.dtype
        emb = self.timestep_embedder(sinusoidal_timestep_embedding(timestep).to(dtype))
        return emb + self.text_embedder(pooled_projection)


class HunyuanVideoPatchEmbed(nn.Module):
    """Non-overlapping 3-D patchify + linear projection.

    The reference uses ``nn.Conv3d(kernel = stride = patch)`` (``layers.py:28-35``).  With
    kernel == stride the convolution is exactly a GEMM over gathered patches, which is
    how it is computed here: ``[B, C, F, H, W] -> [B*S, C*pt*ph*pw] @ W^T``.  The parameter
    keeps the Conv3d name and 5-D shape (``proj.weight [D, C, pt, ph, pw]``).
    """

    def __init__(self, patch_size: Tuple[int, int, int], in_chans: int, embed_dim: int):
        super().__init__()
        self.patch_size = tuple(patch_size)
        self.proj = nn.Conv3d(in_chans, embed_dim, kernel_size=self.patch_size, stride=self.patch_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, C, Fr, H, W = x.shape
        pt, ph, pw = self.patch_size
        f, h, w = Fr // pt, H // ph, W // pw
        patches = x.reshape(B, C, f, pt, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, f * h * w, -1)
        return F.linear(patches, self.proj.weight.reshape(self.proj.weight.shape[0], -1), self.proj.bias)


def rotary_table_1d(dim: int, pos: torch.Tensor, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin of ``pos * theta^(-2j/dim)`` with every frequency repeated twice."""
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=pos.device)[: dim // 2] / dim))
    ang = torch.outer(pos.float(), freqs)
    return ang.cos().repeat_interleave(2, dim=1), ang.sin().repeat_interleave(2, dim=1)


class HunyuanVideoRotaryPosEmbed(nn.Module):
    """3-axis (t, h, w) rotary table ``[S, head_dim]`` in fp32 (``layers.py:209-252``)."""

    def __init__(self, patch_size: int, patch_size_t: int, rope_dim: Sequence[int], theta: float = 256.0):
        super().__init__()
        self.patch_size, self.patch_size_t = patch_size, patch_size_t
        self.rope_dim, self.theta = tuple(rope_dim), theta
        self._cache = {}

    def forward(self, hidden_states: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        _, _, Fr, H, W = hidden_states.shape
        sizes = (Fr // self.patch_size_t, H // self.patch_size, W // self.patch_size)
        key = (sizes, hidden_states.device)
        hit = self._cache.get(key)
        if hit is not None:
            return hit
        grids = torch.meshgrid(*[torch.arange(n, dtype=torch.float32, device=hidden_states.device) for n in sizes],
                               indexing="ij")
        cos, sin = [], []
        for i in range(3):
            c, s = rotary_table_1d(self.rope_dim[i], grids[i].reshape(-1), self.theta)
            cos.append(c)
            sin.append(s)
        out = (torch.cat(cos, dim=1), torch.cat(sin, dim=1))
        self._cache = {key: out}      # one entry: the table depends only on the latent shape
        return out
