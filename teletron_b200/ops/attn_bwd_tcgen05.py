"""Python side of the tcgen05 attention backward (``csrc/attn_bwd_tcgen05.cu``) after a row-dot preprocess.

Two variants:

* ``fused`` (default): one key-stationary kernel computes the scores once and forms dK, dV and this key tile's dQ
  contribution (five products per tile pair); dQ is accumulated in an fp32 scratch with vector reductions, then scaled
  and rounded to bf16.  The order of those additions is not fixed, so dQ is reproducible to fp32 rounding only.
* ``split`` (``TELETRON_B200_ATTN_BWD_FUSED=0``, or :func:`set_fused`): two deterministic, atomics-free kernels
  (key-stationary for dK / dV, query-stationary for dQ; seven products per tile pair).
"""

from __future__ import annotations

import os

import torch

from . import _lib
from ._lib import c_float, c_int, call, check, ptr, stream
from .gemm_tcgen05 import status_tensor

BF16 = torch.bfloat16
_FUSED = os.environ.get("TELETRON_B200_ATTN_BWD_FUSED", "1") != "0"
COUNTERS = {"fused": 0, "split": 0}
_SCRATCH: dict = {}


def set_fused(on: bool) -> bool:
    """Select the one-pass (True) or the two-kernel deterministic (False) backward; returns the previous setting."""
    global _FUSED
    was, _FUSED = _FUSED, bool(on)
    return was


def _dq_scratch(device, numel: int) -> torch.Tensor:
    """fp32 accumulator for dQ, kept per device and grown on demand (the launcher zeroes the part it uses)."""
    buf = _SCRATCH.get(device)
    if buf is None or buf.numel() < numel:
        _SCRATCH.pop(device, None)
        buf = _SCRATCH[device] = torch.empty(numel, dtype=torch.float32, device=device)
    return buf


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
    if _FUSED:
        COUNTERS["fused"] += 1
        acc = _dq_scratch(q.device, B * H * ((S + 127) // 128 * 128) * D)
        call("tt_attn_bwd_fused", ptr(q), ptr(k), ptr(v), ptr(out), ptr(dout), ptr(lse), ptr(delta), ptr(acc), ptr(dq), ptr(dk),
             ptr(dv), c_int(B), c_int(H), c_int(S), c_int(kv_len), c_int(mask_range[0]), c_int(mask_range[1]), c_int(pitch),
             c_float(scale), ptr(status_tensor(q.device)), stream())
        return dq, dk, dv
    COUNTERS["split"] += 1
    call("tt_attn_bwd", ptr(q), ptr(k), ptr(v), ptr(out), ptr(dout), ptr(lse), ptr(delta), ptr(dq), ptr(dk), ptr(dv),
         c_int(B), c_int(H), c_int(S), c_int(kv_len), c_int(mask_range[0]), c_int(mask_range[1]), c_int(pitch), c_float(scale),
         ptr(status_tensor(q.device)), stream())
    return dq, dk, dv
