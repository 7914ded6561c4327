"""Python side of the tcgen05 attention backward (``csrc/attn_bwd_tcgen05.cu``): two deterministic,
atomics-free kernels (key-stationary for dK / dV, query-stationary for dQ) after a row-dot preprocess."""

from __future__ import annotations

import torch

from . import _lib
from ._lib import c_float, c_int, call, check, ptr, stream
from .gemm_tcgen05 import status_tensor

BF16 = torch.bfloat16


def supported(q: torch.Tensor) -> bool:
    return _lib.available() and q.is_cuda and q.dtype == BF16 and q.dim() == 4 and q.shape[-1] == 128


def backward(dout, q, k, v, out, lse, scale: float, kv_len: int, outs=None, mask_range=(0, 0)):
    """``outs``: optional ``(dq, dk, dv)`` tensors to write into (contiguous, shaped like ``q``), e.g. regions of a
    symmetric heap that peers will read."""
    B, H, S, D = q.shape
    pitch = lse.shape[-1]
    dout = check(dout.contiguous(), BF16, "dout")
    out = check(out, BF16, "out")
    delta = torch.zeros(B, H, pitch, dtype=torch.float32, device=q.device)
    if outs is None:
        dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    else:
        dq, dk, dv = (check(t, BF16, n) for t, n in zip(outs, ("dq", "dk", "dv")))
        if any(t.shape != q.shape for t in (dq, dk, dv)):
            raise _lib.NativeError("gradient outputs must have the shape of q")
    call("tt_attn_bwd", ptr(q), ptr(k), ptr(v), ptr(out), ptr(dout), ptr(lse), ptr(delta), ptr(dq), ptr(dk), ptr(dv),
         c_int(B), c_int(H), c_int(S), c_int(kv_len), c_int(mask_range[0]), c_int(mask_range[1]), c_int(pitch), c_float(scale),
         ptr(status_tensor(q.device)), stream())
    return dq, dk, dv
