"""Synthetic dataset with the shapes of the real pipeline (``teletron/datasets/fake_dataset.py:10-44``).

Each item carries random pixels, a first reference frame, LLaMA-sized prompt embeddings, a pooled
CLIP vector, pre-encoded latents and a prompt string.  Items are a pure function of the index so
resumed / re-sharded runs see the same samples.  ``with_pixels=False`` skips the (large) pixel tensors
for latent-only training and benchmarks; the reference always materialises ``randn(F, 3, H, W)`` on the
CPU, even when only its shape is read (``teletron/training/utils.py:98-110``).
"""

from __future__ import annotations

import random
import string

import torch
from torch.utils.data import Dataset

from .registry import DATASETS


@DATASETS.register_module()
class FakeDataset(Dataset):
    def __init__(self, num_frames: int = 33, video_resolution=(1280, 720), text_len: int = 120,
                 text_dim: int = 4096, pooled_dim: int = 768, latent_channels: int = 16, length: int = 10_000_000,
                 with_pixels: bool = True, seed: int = 0, **_unused):
        self.num_frames = int(num_frames)
        self.width, self.height = int(video_resolution[0]), int(video_resolution[1])
        self.text_len, self.text_dim, self.pooled_dim = text_len, text_dim, pooled_dim
        self.latent_channels, self.length, self.with_pixels, self.seed = latent_channels, length, with_pixels, seed

    def __len__(self):
        return self.length

    def __getitem__(self, idx: int):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + int(idx))
        F, H, W = self.num_frames, self.height, self.width
        item = {
            "prompt_embeds": torch.randn(self.text_len, self.text_dim, generator=g),
            "prompt_attention_mask": torch.ones(self.text_len, dtype=torch.bool),
            "clip_text_embed": torch.randn(self.pooled_dim, generator=g),
            "latents": torch.randn(self.latent_channels, (F - 1) // 4 + 1, H // 8, W // 8, generator=g).to(torch.bfloat16),
        }
        if self.with_pixels:
            item["images"] = torch.randn(F, 3, H, W, generator=g)
            item["first_ref_image"] = torch.randn(3, H, W, generator=g)
        rnd = random.Random(self.seed * 7919 + int(idx))
        item["prompt"] = "".join(rnd.choice(string.ascii_lowercase + " ") for _ in range(880))
        return item
