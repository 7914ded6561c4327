"""Optimizer update op on flat ranges (torch reference + sm_100a kernel dispatch)."""

from __future__ import annotations

from typing import Optional

import torch


def _pack16(master: torch.Tensor):
    """fp32 -> (bf16 weight, int16 remainder).  The weight is the fp32 bit pattern rounded half-up in
    magnitude to its top 16 bits, so the remainder always lies in [-32768, 32767]."""
    bits = master.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    hi = ((bits + 0x8000) >> 16) & 0xFFFF
    lo = bits - (hi << 16)
    hi16 = torch.where(hi >= 0x8000, hi - 0x10000, hi).to(torch.int16)
    return hi16.view(torch.bfloat16), lo.to(torch.int16)


def _unpack16(hi: torch.Tensor, lo: torch.Tensor) -> torch.Tensor:
    hb = hi.contiguous().view(torch.int16).to(torch.int64) & 0xFFFF
    bits = ((hb << 16) + lo.to(torch.int64)) & 0xFFFFFFFF
    bits = torch.where(bits >= 0x80000000, bits - 0x100000000, bits).to(torch.int32)
    return bits.view(torch.float32)


def adamw_update_reference(param, grad, exp_avg, exp_avg_sq, master, master_lo, *, lr, beta1, beta2, eps,
                           weight_decay, step, grad_scale=1.0) -> None:
    g = grad.float() * grad_scale
    if master is not None:
        w = master
    elif master_lo is not None:
        w = _unpack16(param, master_lo)
    else:
        w = param.float()
    m = exp_avg.float().mul_(beta1).add_(g, alpha=1.0 - beta1)
    v = exp_avg_sq.float().mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    update = (m / bc1) / ((v / bc2).sqrt_() + eps)
    w = w * (1.0 - lr * weight_decay) - lr * update
    if master is not None:
        master.copy_(w)
        param.copy_(w)
    elif master_lo is not None:
        hi, lo = _pack16(w.contiguous())
        param.copy_(hi)
        master_lo.copy_(lo)
    else:
        param.copy_(w)
    exp_avg.copy_(m)
    exp_avg_sq.copy_(v)


def adamw_update(param: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor,
                 master: Optional[torch.Tensor], master_lo: Optional[torch.Tensor], *, lr: float, beta1: float,
                 beta2: float, eps: float, weight_decay: float, step: int, grad_scale: float = 1.0) -> None:
    """One AdamW update of a flat range, in place.

    Exactly one of the weight sources is authoritative: ``master`` (fp32), ``master_lo`` (the int16
    remainder that, with the bf16 ``param``, reconstructs an fp32 master exactly) or ``param`` itself.
    """
    from . import _use_cuda
    if param.is_cuda and param.dtype == torch.bfloat16 and _use_cuda(param):
        from . import cuda_ops
        cuda_ops.adamw_update(param, grad, exp_avg, exp_avg_sq, master, master_lo, lr=lr, beta1=beta1, beta2=beta2,
                              eps=eps, weight_decay=weight_decay, step=step, grad_scale=grad_scale)
        return
    adamw_update_reference(param, grad, exp_avg, exp_avg_sq, master, master_lo, lr=lr, beta1=beta1, beta2=beta2,
                           eps=eps, weight_decay=weight_decay, step=step, grad_scale=grad_scale)
