"""Python side of the tcgen05 flash attention (``csrc/attn_fwd_tcgen05.cu`` / ``csrc/attn_bwd_tcgen05.cu``).

Operands are head-major ``[B, h, S, 128]`` bf16; the result is token-major ``[B, S, h * 128]`` and the
forward also returns the per-row log-sum-exp (fp32, natural log; ``[B, h, pitch]`` with ``pitch`` = S rounded up
to 64 and ``+inf`` in the padding) that the backward uses.
"""

from __future__ import annotations

import contextlib
import math
from typing import Optional

import torch

from . import _lib
from ._lib import c_float, c_int, call, check, ptr, stream
from .gemm_tcgen05 import status_tensor

BF16 = torch.bfloat16


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    return (_lib.available() and q.is_cuda and q.dtype == BF16 and q.dim() == 4 and q.shape[-1] == 128
            and q.shape == k.shape == v.shape)


def _mask(mask_range, kv_len: int):
    """Normalised ``(lo, hi)`` of the extra masked key range (``(0, 0)``: none)."""
    if mask_range is None:
        return 0, 0
    lo, hi = int(mask_range[0]), min(int(mask_range[1]), kv_len)
    return (lo, hi) if lo < hi else (0, 0)


def forward(q, k, v, kv_valid_len: Optional[int], scale: Optional[float], mask_range=None):
    """``mask_range = (lo, hi)``: keys in ``[lo, hi)`` are masked in addition to those at and beyond ``kv_valid_len``."""
    B, H, S, D = q.shape
    q, k, v = (check(t.contiguous(), BF16, n) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    out = torch.empty(B, S, H * D, dtype=BF16, device=q.device)
    pitch = (S + 63) // 64 * 64       # the backward reads statistics in aligned chunks of 64 queries
    lse = torch.full((B, H, pitch), float("inf"), dtype=torch.float32, device=q.device)
    kv_len = S if kv_valid_len is None else min(int(kv_valid_len), S)
    sc = (1.0 / math.sqrt(D)) if scale is None else float(scale)
    lo, hi = _mask(mask_range, kv_len)
    call("tt_attn_fwd", ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), c_int(B), c_int(H), c_int(S), c_int(kv_len),
         c_int(lo), c_int(hi), c_int(pitch), c_float(sc), ptr(status_tensor(q.device)), stream())
    return out, lse, q, k, v, sc, kv_len


_CACHE = None
_CACHE_MODE = None


@contextlib.contextmanager
def attention_cache(store: list, mode: str):
    """``mode="record"``: append every attention call's (out, lse) to ``store``; ``mode="replay"``: consume them in the
    same order instead of running the forward kernel (used by the block checkpoint that keeps attention outputs)."""
    global _CACHE, _CACHE_MODE
    prev = (_CACHE, _CACHE_MODE)
    _CACHE, _CACHE_MODE = store, mode
    try:
        yield
    finally:
        _CACHE, _CACHE_MODE = prev


def _forward_cached(q, k, v, kv_valid_len, scale, mask_range=None):
    if _CACHE_MODE == "replay" and _CACHE:
        out, lse = _CACHE.pop(0)
        B, H, S, D = q.shape
        q, k, v = (check(t.contiguous(), BF16, n) for t, n in ((q, "q"), (k, "k"), (v, "v")))
        sc = (1.0 / math.sqrt(D)) if scale is None else float(scale)
        kv_len = S if kv_valid_len is None else min(int(kv_valid_len), S)
        return out, lse, q, k, v, sc, kv_len
    res = forward(q, k, v, kv_valid_len, scale, mask_range)
    if _CACHE_MODE == "record":
        _CACHE.append((res[0], res[1]))
    return res


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, kv_valid_len, scale, mask_range=None):
        out, lse, qc, kc, vc, sc, kv_len = _forward_cached(q, k, v, kv_valid_len, scale, mask_range)
        ctx.save_for_backward(qc, kc, vc, out, lse)
        ctx.sc, ctx.kv_len, ctx.mask = sc, kv_len, _mask(mask_range, kv_len)
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import attn_backward
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = attn_backward.backward(dout.contiguous(), q, k, v, out, lse, ctx.sc, ctx.kv_len, mask_range=ctx.mask)
        return dq, dk, dv, None, None, None


def attention(q, k, v, kv_valid_len=None, scale=None, mask_range=None):
    return _Attention.apply(q, k, v, kv_valid_len, scale, mask_range)
