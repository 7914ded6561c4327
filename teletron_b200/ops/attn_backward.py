"""Attention backward given the forward's output and log-sum-exp.

``backward(dout [B, S, h*128], q, k, v [B, h, S, 128], out [B, S, h*128], lse [B, h, S])`` returns
``dq, dk, dv`` in the head-major layout of the inputs.  Backend ``tcgen05`` is the hand-written kernel;
``flash`` calls the flash-attention library's backward on the same (out, lse) pair and is the fallback
for cases the kernel does not take.
"""

from __future__ import annotations

import os

import torch

_BACKEND = os.environ.get("TELETRON_B200_ATTN_BWD", "auto")
COUNTERS = {"tcgen05": 0, "flash": 0, "recompute": 0}


def _library_fallback(what: str, t: torch.Tensor) -> None:
    from . import fallback
    fallback.note(what, f"q {tuple(t.shape)} {t.dtype}")


def _flash(dout, q, k, v, out, lse, scale):
    from flash_attn.flash_attn_interface import _flash_attn_backward
    B, H, S, D = q.shape
    dq, dk, dv = (torch.empty(B, H, S, D, dtype=q.dtype, device=q.device) for _ in range(3))
    _flash_attn_backward(dout.view(B, S, H, D), q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                         out.view(B, S, H, D), lse[..., :S].contiguous(), dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2),
                         0.0, scale, False, -1, -1, 0.0, None, False, None)
    return dq, dk, dv


def _recompute(dout, q, k, v, scale, kv_len, mask_range=None):
    """Reference-grade fallback: differentiate the PyTorch attention (used for masked keys)."""
    from . import reference
    with torch.enable_grad():
        qq, kk, vv = (t.detach().requires_grad_() for t in (q, k, v))
        o = reference.attention(qq, kk, vv, kv_len if kv_len < q.shape[2] else None, scale, mask_range)
        return torch.autograd.grad(o, (qq, kk, vv), dout)


def backward(dout, q, k, v, out, lse, scale: float, kv_len: int, outs=None, mask_range=(0, 0)):
    """``outs``: optional ``(dq, dk, dv)`` destinations (only the tcgen05 kernel writes in place; the library fallbacks
    copy into them)."""
    S = q.shape[2]
    if _BACKEND in ("auto", "tcgen05"):
        from . import attn_bwd_tcgen05
        if attn_bwd_tcgen05.supported(q):
            COUNTERS["tcgen05"] += 1
            return attn_bwd_tcgen05.backward(dout, q, k, v, out, lse, scale, kv_len, outs, mask_range or (0, 0))
        if _BACKEND == "tcgen05":
            raise RuntimeError("tcgen05 attention backward unavailable")
    _library_fallback("attention backward", q)
    if kv_len < S or (mask_range and mask_range[0] < mask_range[1]):
        COUNTERS["recompute"] += 1
        res = _recompute(dout, q, k, v, scale, kv_len, mask_range)
    else:
        COUNTERS["flash"] += 1
        res = _flash(dout, q, k, v, out, lse, scale)
    if outs is not None:
        for dst, src in zip(outs, res):
            dst.copy_(src)
        return tuple(outs)
    return res
