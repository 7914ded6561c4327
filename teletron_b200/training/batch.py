"""Per-step batch distribution inside a TP x CP block.

The first rank of every TP x CP block fetches the sample - from its dataloader or, in
encoder-service mode, from its producer rank - and shares it with the block
(``teletron/training/utils.py:77-230``).  The reference ships the tensor sizes with
``broadcast_object_list`` (pickle -> CPU -> GPU -> NCCL, a blocking host sync every step) and, in
its default mode, broadcasts raw fp32 pixels so every rank re-runs the VAE (``:202-221``).  Here the
shapes travel in one fixed-size int64 header tensor, and only model inputs (latents + embeddings) are
ever broadcast: when pixels are present the source rank encodes them first.
"""

from __future__ import annotations

from typing import Dict, Iterator, Optional

import torch
import torch.distributed as dist

from ..parallel import state as ps

# fixed key order: header row i describes key i
BATCH_KEYS = ("latents", "prompt_embeds", "prompt_attention_mask", "clip_text_embed", "first_frame_latents")
_DTYPES = (torch.float32, torch.bfloat16, torch.float16, torch.bool, torch.int64, torch.int32)
_MAX_DIMS = 6


def _encode_header(batch: Dict[str, torch.Tensor], device) -> torch.Tensor:
    h = torch.zeros(len(BATCH_KEYS), 2 + _MAX_DIMS, dtype=torch.int64)
    for i, k in enumerate(BATCH_KEYS):
        t = batch.get(k)
        if t is None:
            continue
        h[i, 0] = 1 + _DTYPES.index(t.dtype)
        h[i, 1] = t.dim()
        for j, d in enumerate(t.shape):
            h[i, 2 + j] = d
    return h.to(device)


def _decode_header(h: torch.Tensor):
    h = h.cpu()
    out = {}
    for i, k in enumerate(BATCH_KEYS):
        if int(h[i, 0]) == 0:
            continue
        nd = int(h[i, 1])
        out[k] = (_DTYPES[int(h[i, 0]) - 1], tuple(int(x) for x in h[i, 2:2 + nd]))
    return out


def broadcast_batch(batch: Optional[Dict[str, torch.Tensor]], device, group=None, src: Optional[int] = None):
    """Broadcast ``batch`` (given on the source rank, ``None`` elsewhere) over the TP x CP block."""
    group = ps.get_tensor_context_parallel_group() if group is None else group
    if group is None or dist.get_world_size(group) == 1:
        return {k: v.to(device, non_blocking=True) for k, v in batch.items() if isinstance(v, torch.Tensor) and k in BATCH_KEYS}
    src = ps.get_tensor_context_parallel_src_rank() if src is None else src
    is_src = dist.get_rank() == src
    header = _encode_header(batch, device) if is_src else torch.zeros(len(BATCH_KEYS), 2 + _MAX_DIMS, dtype=torch.int64, device=device)
    dist.broadcast(header, src=src, group=group)
    out = {}
    for k, (dtype, shape) in _decode_header(header).items():
        if is_src:
            t = batch[k].to(device, non_blocking=True).contiguous()
        else:
            t = torch.empty(shape, dtype=dtype, device=device)
        if dtype == torch.bool:
            tb = t.to(torch.uint8)
            dist.broadcast(tb, src=src, group=group)
            t = tb.bool()
        else:
            dist.broadcast(t, src=src, group=group)
        out[k] = t
    return out


def get_batch_on_this_tp_cp_rank(data_iterator: Optional[Iterator], device, consumer=None, encode_fn=None):
    """One sample for this rank.

    ``data_iterator`` is consulted on the TP x CP source rank only.  ``consumer`` (an
    :class:`teletron_b200.encoder_service.EncoderConsumer`) replaces it in encoder-service mode.
    ``encode_fn(images) -> latents`` is applied on the source rank when the sample has pixels but
    no latents.
    """
    group = ps.get_tensor_context_parallel_group()
    is_src = group is None or dist.get_rank() == ps.get_tensor_context_parallel_src_rank()
    batch = None
    if is_src:
        if consumer is not None:
            batch = consumer.next_batch()
        else:
            if data_iterator is None:
                raise RuntimeError("the TP x CP source rank has no data iterator")
            batch = next(data_iterator)
        if batch.get("latents") is None and batch.get("images") is not None:
            if encode_fn is None:
                raise RuntimeError("sample has pixels but no latents and no VAE is available")
            batch = dict(batch)
            batch["latents"] = encode_fn(batch["images"].to(device))
            if batch.get("first_ref_image") is not None and batch.get("first_frame_latents") is None:
                batch["first_frame_latents"] = encode_fn(batch["first_ref_image"].to(device)[:, None])
    return broadcast_batch(batch, device, group)


def get_batch_on_this_tp_cp_rank_vast(data_iterator, max_length: int = 256):
    """Entry point with the reference's name (``teletron/training/utils.py:77-82``): takes the device, the encoder-service
    consumer (when ``--distributed-vae``) and the VAE encode function from the global arguments."""
    from .args import get_args
    args = get_args()
    return get_batch_on_this_tp_cp_rank(data_iterator, args.device, consumer=getattr(args, "encoder_consumer", None),
                                        encode_fn=getattr(args, "vae_encode_fn", None))
