"""Attention entry point of the CUDA op layer.

``attention(q, k, v)`` takes head-major ``[B, h, S, 128]`` bf16 operands (the layout the QKV kernel
writes) and returns token-major ``[B, S, h * 128]`` (the layout the output projection reads).
Backend ``tcgen05`` is the hand-written flash attention (``csrc/attn_tcgen05.cu``); backend ``sdpa``
is the library path (``torch`` SDPA, cuDNN / flash backends), which is what the reference runs
(``teletron/models/dit/dit_attention.py:313``) and the fallback for shapes the kernel does not take.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn.functional as F

_BACKEND = os.environ.get("TELETRON_B200_ATTN", "auto")
COUNTERS = {"tcgen05": 0, "sdpa": 0}


def set_backend(name: str) -> None:
    global _BACKEND
    if name not in ("auto", "tcgen05", "sdpa"):
        raise ValueError(name)
    _BACKEND = name


def _sdpa(q, k, v, kv_valid_len, scale, mask_range=None):
    COUNTERS["sdpa"] += 1
    from . import reference
    return reference.attention(q, k, v, kv_valid_len, scale, mask_range)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kv_valid_len: Optional[int] = None,
              scale: Optional[float] = None, mask_range=None) -> torch.Tensor:
    if _BACKEND != "sdpa":
        from . import attn_tcgen05
        if attn_tcgen05.supported(q, k, v):
            COUNTERS["tcgen05"] += 1
            return attn_tcgen05.attention(q, k, v, kv_valid_len, scale, mask_range)
        if _BACKEND == "tcgen05":
            raise RuntimeError(f"tcgen05 attention does not take q {tuple(q.shape)}")
        if q.is_cuda and q.dtype == torch.bfloat16:
            from . import fallback
            fallback.note("attention", f"q {tuple(q.shape)} {q.dtype}")
    return _sdpa(q, k, v, kv_valid_len, scale, mask_range)
