"""Wire format of the encoder-rank -> DiT-rank stream.

One message per training sample, a single flat bf16 tensor (the reference packs
``[len, llama 256x4096 padded, clip 768, first-frame latent, video latent]`` the same way,
``teletron/models/hunyuanvideo/producer.py:199-207``, decoded at ``teletron/training/utils.py:105-130``).
Additions: a 16-slot header of 16-bit integers (bit-cast into the bf16 buffer) carrying a magic
number, a sequence number, the valid text length and the latent geometry, so that the receiver can
size its buffer from flags alone, detect a corrupt or out-of-order message and resynchronise with a
restarted producer.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, Tuple

import torch

HEADER_SLOTS = 16
MAGIC = 0x5443          # "TC"


class ProtocolError(RuntimeError):
    pass


@dataclasses.dataclass(frozen=True)
class MessageSpec:
    """Static geometry of a message, derived from the training flags on both sides."""
    max_text_len: int
    text_dim: int
    pooled_dim: int
    latent_channels: int
    latent_frames: int
    latent_h: int
    latent_w: int

    @staticmethod
    def from_flags(num_frames: int, video_resolution, max_text_len: int = 256, text_dim: int = 4096,
                   pooled_dim: int = 768, latent_channels: int = 16) -> "MessageSpec":
        W, H = int(video_resolution[0]), int(video_resolution[1])
        return MessageSpec(max_text_len, text_dim, pooled_dim, latent_channels, (num_frames - 1) // 4 + 1, H // 8, W // 8)

    @property
    def sizes(self) -> Tuple[int, int, int, int]:
        first = self.latent_channels * self.latent_h * self.latent_w
        return (self.max_text_len * self.text_dim, self.pooled_dim, first, first * self.latent_frames)

    @property
    def numel(self) -> int:
        return HEADER_SLOTS + sum(self.sizes)

    @property
    def nbytes(self) -> int:
        return self.numel * 2


def _header(seq: int, text_len: int, spec: MessageSpec) -> torch.Tensor:
    h = torch.zeros(HEADER_SLOTS, dtype=torch.int16)
    vals = [MAGIC, seq & 0x7FFF, (seq >> 15) & 0x7FFF, text_len, spec.latent_frames, spec.latent_h, spec.latent_w,
            spec.latent_channels, spec.max_text_len, spec.pooled_dim]
    for i, v in enumerate(vals):
        h[i] = v
    checksum = sum(vals) & 0x7FFF
    h[HEADER_SLOTS - 1] = checksum
    return h


def pack_message(spec: MessageSpec, seq: int, prompt_embeds: torch.Tensor, clip_embed: torch.Tensor,
                 first_frame_latent: torch.Tensor, latents: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """``prompt_embeds [L<=max, text_dim]``, ``clip_embed [pooled]``, ``first_frame_latent [C, 1, h, w]``,
    ``latents [C, f, h, w]`` -> flat bf16 message on the latents' device."""
    dev = latents.device
    msg = out if out is not None else torch.empty(spec.numel, dtype=torch.bfloat16, device=dev)
    L = prompt_embeds.shape[0]
    if L > spec.max_text_len:
        raise ProtocolError(f"prompt of {L} tokens exceeds the message capacity {spec.max_text_len}")
    n_text, n_pool, n_first, n_lat = spec.sizes
    if latents.numel() != n_lat or first_frame_latent.numel() != n_first:
        raise ProtocolError(f"latent geometry {tuple(latents.shape)} does not match {spec}")
    msg[:HEADER_SLOTS].view(torch.int16).copy_(_header(seq, L, spec))
    o = HEADER_SLOTS
    text = msg[o:o + n_text].view(spec.max_text_len, spec.text_dim)
    text[:L].copy_(prompt_embeds)
    text[L:].zero_()
    o += n_text
    msg[o:o + n_pool].copy_(clip_embed.reshape(-1))
    o += n_pool
    msg[o:o + n_first].copy_(first_frame_latent.reshape(-1))
    o += n_first
    msg[o:o + n_lat].copy_(latents.reshape(-1))
    return msg


def unpack_message(spec: MessageSpec, msg: torch.Tensor, expect_seq: int = None) -> Dict[str, torch.Tensor]:
    """Views into ``msg`` (no copies) with a leading batch dimension of 1, plus ``seq`` / ``text_len``."""
    h = msg[:HEADER_SLOTS].view(torch.int16).cpu().tolist()
    if h[0] != MAGIC or (sum(h[:10]) & 0x7FFF) != h[HEADER_SLOTS - 1]:
        raise ProtocolError("corrupt message header")
    seq = h[1] | (h[2] << 15)
    if (h[4], h[5], h[6], h[7]) != (spec.latent_frames, spec.latent_h, spec.latent_w, spec.latent_channels):
        raise ProtocolError(f"message geometry {h[4:8]} does not match the receiver's flags {spec}")
    if expect_seq is not None and seq != expect_seq:
        raise ProtocolError(f"out-of-order message: got sequence {seq}, expected {expect_seq}")
    L = h[3]
    n_text, n_pool, n_first, n_lat = spec.sizes
    o = HEADER_SLOTS
    text = msg[o:o + n_text].view(1, spec.max_text_len, spec.text_dim)
    o += n_text
    pooled = msg[o:o + n_pool].view(1, n_pool)
    o += n_pool
    first = msg[o:o + n_first].view(1, spec.latent_channels, 1, spec.latent_h, spec.latent_w)
    o += n_first
    lat = msg[o:o + n_lat].view(1, spec.latent_channels, spec.latent_frames, spec.latent_h, spec.latent_w)
    mask = torch.zeros(1, spec.max_text_len, dtype=torch.bool, device=msg.device)
    mask[:, :L] = True
    return {"seq": seq, "text_len": L, "prompt_embeds": text, "prompt_attention_mask": mask,
            "clip_text_embed": pooled, "first_frame_latents": first, "latents": lat}
