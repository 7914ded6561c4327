"""Text / image -> video sampling with the trained MMDiT (flow-match Euler).

Capabilities of the reference's diffusers-style pipeline (``examples/hunyuanvideo/pipelines.py:575-1016``):
LLaMA prompt template with the instruction prefix cropped off (``:69-80, 275-350``), CLIP pooled prompt (``:352-397``),
flow-match Euler loop with a shifted sigma schedule, I2V first-frame conditioning by channel concatenation
(``:819-836``), token-replace mode with optional first + last frame (``:838-865``), true classifier-free guidance with
the CFG-zero-star rescaling (``:954-969``), embedded guidance, VAE decode (``:1001-1006``).

It is an ``nn.Module``-free orchestrator over components that this package owns: the transformer, the VAE and the
two text encoders (:mod:`teletron_b200.models`).  Frames come back as a ``[B, F, 3, H, W]`` tensor in ``[0, 1]``;
:func:`save_video_tensor` writes them as a video file (:mod:`teletron_b200.inference.video_io`: ``.avi`` with no
dependency, ``.mp4`` through OpenCV, ``.gif``) or as ``.pt`` / ``.npy``.
"""

from __future__ import annotations

import dataclasses
from typing import Callable, List, Optional, Sequence, Union

import torch
import torch.nn.functional as F

DEFAULT_PROMPT_TEMPLATE = {
    "template": (
        "<|start_header_id|>system<|end_header_id|>\n\nDescribe the video by detailing the following aspects: "
        "1. The main content and theme of the video."
        "2. The color, shape, size, texture, quantity, text, and spatial relationships of the objects."
        "3. Actions, events, behaviors temporal relationships, physical movement changes of the objects."
        "4. background environment, light, style and atmosphere."
        "5. camera angles, movements, and transitions used in the video:<|eot_id|>"
        "<|start_header_id|>user<|end_header_id|>\n\n{}<|eot_id|>"
    ),
    "crop_start": 95,
}


@dataclasses.dataclass
class PipelineOutput:
    frames: torch.Tensor          # [B, F, 3, H, W] in [0, 1] (or latents when output_type="latent")


def optimized_scale(positive_flat: torch.Tensor, negative_flat: torch.Tensor) -> torch.Tensor:
    """CFG-zero-star projection coefficient ``<pos, neg> / ||neg||^2`` per sample."""
    dot = (positive_flat.float() * negative_flat.float()).sum(dim=1, keepdim=True)
    sq = negative_flat.float().pow(2).sum(dim=1, keepdim=True) + 1e-8
    return dot / sq


def flow_sigmas(num_steps: int, shift: float = 7.0, device=None) -> torch.Tensor:
    """``num_steps + 1`` sigmas from 1 to 0 with the time shift ``s' = k s / (1 + (k - 1) s)``."""
    s = torch.linspace(1.0, 0.0, num_steps + 1, device=device, dtype=torch.float32)
    return shift * s / (1 + (shift - 1) * s)


def save_video_tensor(frames: torch.Tensor, path: str, fps: float = 15.0) -> str:
    """``frames [F, 3, H, W]`` in ``[0, 1]`` -> file chosen by the extension; returns the path written."""
    from .video_io import export_to_video
    return export_to_video(frames, path, fps)


class HunyuanVideoPipeline:
    def __init__(self, transformer, vae, text_encoder, clip_encoder, flow_shift: float = 7.0,
                 vae_scaling_factor: float = 0.476986):
        self.transformer, self.vae = transformer, vae
        self.text_encoder, self.clip_encoder = text_encoder, clip_encoder
        self.flow_shift, self.vae_scaling_factor = flow_shift, vae_scaling_factor

    @classmethod
    def from_pretrained(cls, base_model_path: Optional[str] = None, transformer_model_path: Optional[str] = None,
                        torch_dtype=torch.bfloat16, device=None, cfg=None, **kw) -> "HunyuanVideoPipeline":
        """Build every component; weights are loaded when paths are given (TeleTron checkpoint directory for the
        transformer, HF directories ``text_encoder`` / ``text_encoder_2`` / ``vae`` under ``base_model_path``)."""
        import os
        from ..models.hunyuanvideo import HunyuanVideoTransformer3DModel, hunyuan_13b
        from ..models.text_encoders import ClipTextEncoder, LlamaTextEncoder
        from ..models.vae import AutoencoderKLHunyuanVideo
        sd = None
        if transformer_model_path:
            from ..convert_ckpt.hunyuan.convert_hunyuanvideo import load_tel_checkpoint, merge_shards
            base = cfg or hunyuan_13b()
            sd = merge_shards(load_tel_checkpoint(transformer_model_path), base.hidden_size, base.mlp_hidden)
        if cfg is None:
            # 33 input channels for first-frame-conditioned (i2v) weights, 16 otherwise: read from the checkpoint when there
            # is one, else from the ``in_channels`` keyword
            w = None if sd is None else sd.get("x_embedder.proj.weight")
            cfg = hunyuan_13b(in_channels=int(w.shape[1]) if w is not None else int(kw.get("in_channels", 16)))
        tr = HunyuanVideoTransformer3DModel(cfg, tp=1, device=device, dtype=torch_dtype).eval()
        if sd is not None:
            tr.load_state_dict(sd, strict=False)
        vae = AutoencoderKLHunyuanVideo().to(device, torch_dtype).eval()
        sub = lambda n: (os.path.join(base_model_path, n) if base_model_path and os.path.isdir(os.path.join(base_model_path, n)) else None)  # noqa: E731
        if sub("vae"):
            from ..convert_ckpt.hunyuan.convert_hunyuanvideo import _load_any
            vae.load_state_dict(_load_any(sub("vae")), strict=False)
        llama = LlamaTextEncoder(sub("text_encoder"), 256 + DEFAULT_PROMPT_TEMPLATE["crop_start"], device, torch_dtype, config=kw.get("llama_config"))
        clip = ClipTextEncoder(sub("text_encoder_2"), 77, device, torch_dtype, config=kw.get("clip_config"))
        return cls(tr, vae, llama, clip)

    # ---- prompt ---------------------------------------------------------------------------
    def encode_prompt(self, prompt: Sequence[str], template=DEFAULT_PROMPT_TEMPLATE, max_sequence_length: int = 256):
        crop = template["crop_start"]
        texts = [template["template"].format(p) for p in prompt]
        self.text_encoder.max_length = max_sequence_length + crop
        emb, mask = self.text_encoder(texts)
        if self.text_encoder.tokenizer is not None:       # real tokenizer: drop the instruction prefix
            emb, mask = emb[:, crop:], mask[:, crop:]
        else:                                              # stand-in tokenizer: the prefix length is not 95 tokens
            emb, mask = emb[:, :max_sequence_length], mask[:, :max_sequence_length]
        pooled = self.clip_encoder(list(prompt))
        return emb, mask, pooled

    # ---- sampling -------------------------------------------------------------------------
    @torch.no_grad()
    def __call__(self, prompt: Union[str, List[str]], negative_prompt: str = "", height: int = 720, width: int = 1280,
                 num_frames: int = 129, num_inference_steps: int = 50, guidance_scale: float = 6.0,
                 embedded_guidance_scale: float = 1.0, model_type: str = "t2v", ref_images: Optional[torch.Tensor] = None,
                 first_last: bool = False, cfg_zero_star: bool = False, seed: int = -1,
                 generator: Optional[torch.Generator] = None, latents: Optional[torch.Tensor] = None,
                 output_type: str = "pt", max_sequence_length: int = 256,
                 callback_on_step_end: Optional[Callable] = None) -> PipelineOutput:
        """``ref_images``: ``[F_ref, 3, H, W]`` in ``[-1, 1]`` (first frame used for ``i2v``; first / last for ``token_replace``)."""
        if model_type not in ("t2v", "i2v", "token_replace"):
            raise ValueError(f"unknown model_type {model_type}")
        prompts = [prompt] if isinstance(prompt, str) else list(prompt)
        B = len(prompts)
        p0 = next(self.transformer.parameters())
        dev, dtype = p0.device, p0.dtype
        if generator is None:
            generator = torch.Generator(device=dev)
            generator.manual_seed(seed if seed >= 0 else torch.seed() % (2 ** 31))
        do_cfg = guidance_scale > 1.0
        emb, mask, pooled = self.encode_prompt(prompts, max_sequence_length=max_sequence_length)
        if do_cfg:
            nemb, nmask, npooled = self.encode_prompt([negative_prompt] * B, max_sequence_length=max_sequence_length)
        f = (num_frames - 1) // 4 + 1
        shape = (B, 16, f, height // 8, width // 8)
        if latents is None:
            latents = torch.randn(shape, generator=generator, device=dev, dtype=torch.float32).to(dtype)
        cond = mask_lat = first_lat = last_lat = None
        if ref_images is not None:
            ref = ref_images.to(dev, dtype)
            # the posterior sample of a reference frame is drawn from the call's generator (the reference draws it from the
            # global RNG, examples/hunyuanvideo/pipelines.py:824-826, so a fixed seed did not fix the video)
            enc = lambda img: self.vae.encode(img.unsqueeze(0).permute(0, 2, 1, 3, 4), generator=generator) * self.vae_scaling_factor  # noqa: E731
            if model_type == "i2v":
                first = enc(ref[:1]).to(dtype)
                cond = F.pad(first, (0, 0, 0, 0, 0, f - first.shape[2])).expand(B, -1, -1, -1, -1)
                mask_lat = torch.zeros(B, 1, f, shape[3], shape[4], device=dev, dtype=dtype)
                mask_lat[:, :, 0] = 1
            elif model_type == "token_replace":
                first_lat = enc(ref[:1]).to(dtype).expand(B, -1, -1, -1, -1)
                if first_last:
                    last_lat = enc(ref[-1:]).to(dtype).expand(B, -1, -1, -1, -1)
        if model_type == "i2v" and cond is None:
            raise ValueError("model_type='i2v' needs ref_images")

        def replace_tokens(x):
            if first_lat is None:
                return x
            parts = [first_lat, x[:, :, 1:-1] if last_lat is not None else x[:, :, 1:]]
            if last_lat is not None:
                parts.append(last_lat)
            return torch.cat(parts, dim=2)

        latents = replace_tokens(latents)
        sigmas = flow_sigmas(num_inference_steps, self.flow_shift, dev)
        guidance = torch.full((B,), embedded_guidance_scale * 1000.0, device=dev, dtype=torch.float32)
        for i in range(num_inference_steps):
            t = (sigmas[i] * 1000.0).expand(B)
            x_in = latents if cond is None else torch.cat([latents, cond, mask_lat], dim=1)
            pred = self.transformer(x_in, t, emb.to(dtype), mask, pooled.to(dtype), guidance)[0]
            if do_cfg:
                unc = self.transformer(x_in, t, nemb.to(dtype), nmask, npooled.to(dtype), guidance)[0]
                if cfg_zero_star:
                    if i <= 1:
                        pred = pred * 0
                    else:
                        alpha = optimized_scale(pred.reshape(B, -1), unc.reshape(B, -1)).view(B, 1, 1, 1, 1).to(pred.dtype)
                        pred = unc * alpha + guidance_scale * (pred - unc * alpha)
                else:
                    pred = unc + guidance_scale * (pred - unc)
            latents = (latents.float() + (sigmas[i + 1] - sigmas[i]) * pred.float()).to(dtype)
            latents = replace_tokens(latents)
            if callback_on_step_end is not None:
                out = callback_on_step_end(self, i, t, {"latents": latents})
                if out and "latents" in out:
                    latents = out["latents"]
        if output_type == "latent":
            return PipelineOutput(frames=latents)
        video = self.vae.decode(latents / self.vae_scaling_factor)                     # [B, 3, F, H, W] in [-1, 1]
        frames = (video.float().clamp(-1, 1) * 0.5 + 0.5).permute(0, 2, 1, 3, 4).contiguous()
        return PipelineOutput(frames=frames)
