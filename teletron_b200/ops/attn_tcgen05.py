"""Python side of the tcgen05 flash attention (``csrc/attn_tcgen05.cu``)."""

from __future__ import annotations

import torch

from . import _lib


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    return False


def attention(q, k, v, kv_valid_len=None, scale=None):
    raise _lib.NativeError("tcgen05 attention is not built")
