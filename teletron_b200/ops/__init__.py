"""Functional op layer.

Every op has two implementations behind one signature:

* ``reference`` - pure PyTorch (CPU capable, plain autograd); the numerics oracle and
  the restated library baseline.
* ``cuda`` - hand-written sm_100a kernels from ``teletron_b200/csrc`` reached through
  ``ctypes`` (:mod:`teletron_b200.ops._lib`), wrapped in ``autograd.Function``s.

Selection: :func:`set_impl` (``"auto" | "torch" | "cuda"``).  ``auto`` uses the CUDA
kernels for CUDA bf16 tensors and the reference otherwise.  On a machine with a GPU the
native library must be present: there is no silent fallback (set
``TELETRON_B200_ALLOW_FALLBACK=1`` to opt into one, e.g. for the baseline arm).
"""

from __future__ import annotations

import contextlib
import os

import torch

from . import reference
from . import optim  # noqa: F401

_IMPL = os.environ.get("TELETRON_B200_IMPL", "auto")


def set_impl(name: str) -> None:
    global _IMPL
    if name not in ("auto", "torch", "cuda"):
        raise ValueError(name)
    _IMPL = name


def get_impl() -> str:
    return _IMPL


_NVTX = os.environ.get("TELETRON_B200_NVTX", "0") == "1"


def set_nvtx(enabled: bool) -> None:
    """Named ranges around blocks and steps for a timeline profiler (set by ``--profile``)."""
    global _NVTX
    _NVTX = bool(enabled)


@contextlib.contextmanager
def nvtx_range(name: str):
    """``torch.cuda.nvtx`` range when enabled and CUDA is present; otherwise free."""
    if _NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


@contextlib.contextmanager
def impl(name: str):
    prev = get_impl()
    set_impl(name)
    try:
        yield
    finally:
        set_impl(prev)


def _use_cuda(*tensors: torch.Tensor) -> bool:
    """True when the sm_100a kernels should run for these operands."""
    if _IMPL == "torch":
        return False
    t0 = tensors[0]
    if not t0.is_cuda:
        if _IMPL == "cuda":
            raise RuntimeError("impl='cuda' requested for a non-CUDA tensor")
        return False
    if t0.dtype != torch.bfloat16:
        if _IMPL == "cuda":
            raise RuntimeError("the sm_100a kernels take bf16 operands, got %s" % t0.dtype)
        return False
    from . import _lib
    if not _lib.available():
        if os.environ.get("TELETRON_B200_ALLOW_FALLBACK") == "1" and _IMPL != "cuda":
            return False
        raise RuntimeError(
            "teletron_b200 native library is not built (run `python -m teletron_b200.build`); "
            "refusing to fall back to library kernels on a GPU: " + _lib.load_error())
    return True


def layernorm_modulate(x, scale, shift, eps: float = 1e-6):
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.layernorm_modulate(x, scale, shift, eps)
    return reference.layernorm_modulate(x, scale, shift, eps)


def gate_residual(residual, branch, gate):
    if _use_cuda(residual):
        from . import cuda_ops
        return cuda_ops.gate_residual(residual, branch, gate)
    return reference.gate_residual(residual, branch, gate)


def gate_residual_layernorm_modulate(residual, branch, gate, scale, shift, eps: float = 1e-6):
    if _use_cuda(residual):
        from . import cuda_ops
        return cuda_ops.gate_residual_layernorm_modulate(residual, branch, gate, scale, shift, eps)
    return reference.gate_residual_layernorm_modulate(residual, branch, gate, scale, shift, eps)


def rmsnorm(x, weight, eps: float = 1e-6):
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.rmsnorm(x, weight, eps)
    return reference.rmsnorm(x, weight, eps)


def apply_rope(x, cos, sin):
    return reference.apply_rope(x, cos, sin)


def linear(x, weight, bias=None, activation=None):
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.linear(x, weight, bias, activation)
    return reference.linear(x, weight, bias, activation)


def linear_merged(x1, x2, weight, bias=None):
    """``cat([x1, x2], -1) @ weight^T + bias`` without ever forming the concatenated gradient in the backward."""
    if _use_cuda(x1):
        from . import cuda_ops
        return cuda_ops.linear_merged(x1, x2, weight, bias)
    return reference.linear_merged(x1, x2, weight, bias)


def attention(q, k, v, kv_valid_len=None, scale=None, mask_range=None):
    """``kv_valid_len`` masks the key tail, ``mask_range = (lo, hi)`` one more key range."""
    if _use_cuda(q):
        from . import cuda_ops
        return cuda_ops.attention(q, k, v, kv_valid_len, scale, mask_range)
    return reference.attention(q, k, v, kv_valid_len, scale, mask_range)


def qkv_projection(x, weight, bias, q_norm_weight, k_norm_weight, cos, sin, num_heads,
                   eps: float = 1e-6, rope_len=None):
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.qkv_projection(x, weight, bias, q_norm_weight, k_norm_weight, cos, sin,
                                       num_heads, eps, rope_len)
    return reference.qkv_projection(x, weight, bias, q_norm_weight, k_norm_weight, cos, sin,
                                    num_heads, eps, rope_len)


def joint_qkv_projection(x, weight, bias, q_norm_weight, k_norm_weight, cos, sin, x2, weight2, bias2,
                         q_norm_weight2, k_norm_weight2, num_heads, eps: float = 1e-6):
    """Video stream ``x`` (RoPE applied) and text stream ``x2`` (no RoPE), each with its own weights,
    projected into shared ``[B, heads, S + T, D]`` q / k / v (video tokens first)."""
    if _use_cuda(x) and q_norm_weight.shape[0] == 128:
        from . import cuda_ops
        return cuda_ops.joint_qkv_projection(x, weight, bias, q_norm_weight, k_norm_weight, cos, sin, x2, weight2,
                                             bias2, q_norm_weight2, k_norm_weight2, num_heads, eps)
    return reference.joint_qkv_projection(x, weight, bias, q_norm_weight, k_norm_weight, cos, sin, x2, weight2,
                                          bias2, q_norm_weight2, k_norm_weight2, num_heads, eps)


def _flow_kernel_ok(*tensors) -> bool:
    t0 = tensors[0]
    return (t0.is_cuda and all(t.dtype == torch.bfloat16 and t.shape == t0.shape for t in tensors)
            and (t0.numel() // max(1, t0.shape[0])) % 8 == 0 and _use_cuda(t0))


def flow_match_loss(pred, noise, latents, weight):
    if _flow_kernel_ok(pred, noise, latents):
        from . import cuda_ops
        return cuda_ops.flow_match_loss(pred, noise, latents, weight)
    return reference.flow_match_loss(pred, noise, latents, weight)


def noise_mix(latents, noise, sigma):
    """Model input of a flow-matching step: ``(1 - sigma) * latents + sigma * noise`` with one noise level per sample."""
    if _flow_kernel_ok(latents, noise):
        from . import cuda_ops
        return cuda_ops.noise_mix(latents, noise, sigma)
    return reference.noise_mix(latents, noise, sigma)
