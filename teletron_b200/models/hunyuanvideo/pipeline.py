"""Flow-matching training wrapper around the MMDiT (``teletron/models/hunyuanvideo/pipeline.py:40-239``).

Per step: draw a noise level, broadcast it over the TP x CP group, build
``x_t = (1 - sigma) x0 + sigma * eps``, add the I2V first-frame conditioning
(16 latent + 16 conditioning + 1 mask = 33 channels), run the transformer and return the
weighted MSE against the velocity target ``eps - x0``.

Deliberate differences from the reference: the flow-shift flag is honoured
(``sigma' = k sigma / (1 + (k - 1) sigma)``; the reference parses it and ignores it,
``pipeline.py:64``); noise and noise level are drawn on the TP x CP source rank from a
generator keyed by (seed, step, data-parallel rank) and broadcast, instead of relying on
every rank's RNG staying in lock-step (``pipeline.py:118-121``).
"""

from __future__ import annotations

import dataclasses
import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
from torch import nn

from ... import ops
from ...parallel import state as ps
from .config import HunyuanParams
from .model import HunyuanVideoTransformer3DModel


@dataclasses.dataclass
class FlowConfig:
    """Flow-matching knobs (flags ``--flow-*`` of ``pretrain_hunyuanvideo.py:64-75``)."""
    num_train_timesteps: int = 1000
    shift: float = 1.0
    weighting_scheme: str = "none"        # none | sigma_sqrt | cosmap | logit_normal | mode
    logit_mean: float = 0.0
    logit_std: float = 1.0
    mode_scale: float = 1.29
    guidance_scale: float = 1.0
    sanity_check: bool = False
    model_type: str = "i2v"               # "i2v" (33 input channels) | "t2v" (16)
    vae_scaling_factor: float = 0.476986


class FlowMatchScheduler:
    """Sigma table of a flow-match Euler scheduler: ``linspace(1, N, N)[::-1] / N`` then shifted."""

    def __init__(self, num_train_timesteps: int = 1000, shift: float = 1.0):
        t = torch.linspace(1, num_train_timesteps, num_train_timesteps, dtype=torch.float32).flip(0)
        sig = t / num_train_timesteps
        self.sigmas = shift * sig / (1 + (shift - 1) * sig)
        self.timesteps = self.sigmas * num_train_timesteps
        self.num_train_timesteps = num_train_timesteps


def compute_density_for_timestep_sampling(scheme: str, batch_size: int, logit_mean: float = 0.0,
                                          logit_std: float = 1.0, mode_scale: float = 1.29,
                                          generator: Optional[torch.Generator] = None) -> torch.Tensor:
    if scheme == "logit_normal":
        u = torch.normal(mean=logit_mean, std=logit_std, size=(batch_size,), generator=generator)
        return torch.sigmoid(u)
    u = torch.rand(batch_size, generator=generator)
    if scheme == "mode":
        return 1 - u - mode_scale * (torch.cos(math.pi * u / 2) ** 2 - 1 + u)
    return u


def compute_loss_weighting(scheme: str, sigmas: torch.Tensor) -> torch.Tensor:
    if scheme == "sigma_sqrt":
        return sigmas ** -2.0
    if scheme == "cosmap":
        return 2.0 / (math.pi * (1 - 2 * sigmas + 2 * sigmas ** 2))
    return torch.ones_like(sigmas)


class HunyuanPipeline(nn.Module):
    def __init__(self, cfg: HunyuanParams, flow: Optional[FlowConfig] = None, vae: Optional[nn.Module] = None,
                 device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.flow = flow or FlowConfig()
        want = 33 if self.flow.model_type == "i2v" else 16
        if cfg.in_channels != want and cfg.hidden_size == 3072:
            raise ValueError(f"model_type {self.flow.model_type} needs in_channels={want}, got {cfg.in_channels}")
        self.transformer = HunyuanVideoTransformer3DModel(cfg, device=device, dtype=dtype)
        self.scheduler = FlowMatchScheduler(self.flow.num_train_timesteps, self.flow.shift)
        self.vae = vae            # frozen; None when latents come pre-encoded / from the encoder service
        if vae is not None:
            for p in vae.parameters():
                p.requires_grad_(False)
        self.step = 0

    # -- noise level ---------------------------------------------------------------------
    def _draw(self, batch_size: int, latents_shape, device, dtype):
        """Sigma + noise for this step, identical on every rank of the TP x CP block."""
        group = ps.get_tensor_context_parallel_group()
        is_src = group is None or dist.get_rank() == ps.get_tensor_context_parallel_src_rank()
        seed = self.cfg.seed * 1000003 + self.step * 1009 + ps.get_data_parallel_rank()
        gen = torch.Generator(device="cpu").manual_seed(seed)
        u = compute_density_for_timestep_sampling(self.flow.weighting_scheme, batch_size, self.flow.logit_mean,
                                                  self.flow.logit_std, self.flow.mode_scale, generator=gen)
        idx = (u * self.scheduler.num_train_timesteps).long().clamp_(0, self.scheduler.num_train_timesteps - 1)
        sigma = self.scheduler.sigmas[idx].to(device)
        dgen = torch.Generator(device=device).manual_seed(seed + 1)
        noise = torch.randn(latents_shape, generator=dgen, device=device, dtype=torch.float32).to(dtype)
        if group is not None:
            # the generator already agrees across the block; the broadcast makes that a guarantee
            # (call site X13 of the reference, pipeline.py:34-37)
            dist.broadcast(sigma, src=ps.get_tensor_context_parallel_src_rank(), group=group)
        del is_src
        return sigma, noise

    def forward_vae(self, images: torch.Tensor) -> torch.Tensor:
        """``[B, F, C, H, W]`` pixels -> scaled latents ``[B, 16, f, H/8, W/8]`` (``pipeline.py:228-233``)."""
        with torch.no_grad():
            x = images.permute(0, 2, 1, 3, 4).contiguous()
            return self.vae.encode(x) * self.flow.vae_scaling_factor

    def forward(self, batch: Dict[str, torch.Tensor]) -> List[torch.Tensor]:
        flow = self.flow
        dev = next(self.transformer.parameters()).device
        dtype = next(self.transformer.parameters()).dtype
        with torch.no_grad():
            prompt_embeds = batch["prompt_embeds"].to(dev, dtype)
            pooled = batch["clip_text_embed"].to(dev, dtype)
            mask = batch.get("prompt_attention_mask")
            if mask is None:
                mask = torch.ones(prompt_embeds.shape[:2], dtype=torch.bool, device=dev)
            else:
                mask = mask.to(dev)
            if batch.get("latents") is not None:
                latents = batch["latents"].to(dev, dtype)
            else:
                latents = self.forward_vae(batch["images"].to(dev, dtype)).to(dtype)
            B = latents.shape[0]
            sigma, noise = self._draw(B, latents.shape, dev, dtype)
            timesteps = (sigma * self.scheduler.num_train_timesteps).long()
            noisy = ops.noise_mix(latents, noise, sigma)

            if flow.model_type == "i2v":
                if batch.get("first_frame_latents") is not None:
                    first = batch["first_frame_latents"].to(dev, dtype)
                elif batch.get("first_ref_image") is not None and self.vae is not None:
                    first = self.forward_vae(batch["first_ref_image"].to(dev, dtype)[:, None]).to(dtype)
                else:
                    first = latents[:, :, :1]
                cond = torch.zeros_like(latents)
                cond[:, :, :1] = first[:, :, :1]
                m = torch.zeros(B, 1, *latents.shape[2:], device=dev, dtype=dtype)
                m[:, :, 0] = 1.0
                model_in = torch.cat([noisy, cond, m], dim=1)
            else:
                model_in = noisy
            guidance = torch.full((B,), flow.guidance_scale * 1000.0, device=dev, dtype=torch.float32)

            if flow.sanity_check:
                # deterministic inputs so the loss depends only on weights and the parallel layout
                # (pipeline.py:196-202)
                g = torch.Generator(device="cpu").manual_seed(1234)
                model_in = torch.randn(model_in.shape, generator=g).to(dev, dtype)
                prompt_embeds = torch.randn(prompt_embeds.shape, generator=g).to(dev, dtype)
                pooled = torch.randn(pooled.shape, generator=g).to(dev, dtype)
                timesteps = torch.randint(0, 1000, (B,), generator=g).to(dev)
                mask = torch.ones(prompt_embeds.shape[:2], dtype=torch.bool, device=dev)

        pred = self.transformer(model_in, timesteps, prompt_embeds, mask, pooled, guidance)[0]
        self.step += 1
        if flow.sanity_check:
            return [pred.float().norm()]
        weight = compute_loss_weighting(flow.weighting_scheme, sigma.float())
        return [ops.flow_match_loss(pred, noise, latents, weight)]

    def state_dict_for_save_checkpoint(self, prefix: str = "", keep_vars: bool = False):
        """Transformer weights only, keys without prefix (``pipeline.py:235-237``)."""
        return self.transformer.state_dict(prefix=prefix, keep_vars=keep_vars)
