"""Python side of the tcgen05 attention backward (``csrc/attn_bwd_tcgen05.cu``)."""

from __future__ import annotations

import torch


def supported(q: torch.Tensor) -> bool:
    return False


def backward(dout, q, k, v, out, lse, scale, kv_len):
    raise NotImplementedError
