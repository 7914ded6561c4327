"""bf16 GEMM entry points used by the CUDA op layer.

Three operand layouts cover forward, data-gradient and weight-gradient products:

* ``gemm_nt(a [M, K], b [N, K])   -> a @ b.T``   (forward: activations x weight rows)
* ``gemm_nn(a [M, K], b [K, N])   -> a @ b``     (dgrad: output grads x weight)
* ``gemm_tn(a [K, M], b [K, N])   -> a.T @ b``   (wgrad: output grads^T x activations)

Backend ``tcgen05`` is the hand-written sm_100a kernel (``csrc/gemm_tcgen05.cu``: TMA-fed
128B-swizzled shared-memory ring, ``tcgen05.mma`` with TMEM accumulators, fused bias epilogue);
backend ``cublas`` (``torch.matmul``) is the library baseline and the fallback for shapes the kernel
does not take.  Select with ``TELETRON_B200_GEMM`` or :func:`set_backend`.
"""

from __future__ import annotations

import os
from typing import Optional

import torch

_BACKEND = os.environ.get("TELETRON_B200_GEMM", "auto")
COUNTERS = {"tcgen05": 0, "cublas": 0}


def set_backend(name: str) -> None:
    global _BACKEND
    if name not in ("auto", "tcgen05", "cublas"):
        raise ValueError(name)
    _BACKEND = name


def get_backend() -> str:
    return _BACKEND


def _native(a: torch.Tensor, b: torch.Tensor, layout: str, bias: Optional[torch.Tensor]):
    if _BACKEND == "cublas":
        return None
    from . import gemm_tcgen05
    if not gemm_tcgen05.supported(a, b, layout):
        if _BACKEND == "tcgen05":
            raise RuntimeError(f"tcgen05 GEMM does not take {layout} {tuple(a.shape)} x {tuple(b.shape)}")
        if a.is_cuda and a.dtype == torch.bfloat16:
            from . import fallback
            if not fallback.vector_shaped(*a.shape, *b.shape):
                fallback.note("gemm", f"{layout} {tuple(a.shape)} x {tuple(b.shape)} strides {a.stride()} {b.stride()}")
        return None
    COUNTERS["tcgen05"] += 1
    return gemm_tcgen05.gemm(a, b, layout, bias)


def gemm_nt(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    out = _native(a, b, "nt", bias)
    if out is not None:
        return out
    COUNTERS["cublas"] += 1
    return torch.nn.functional.linear(a, b, bias)


def gemm_nn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    out = _native(a, b, "nn", None)
    if out is not None:
        return out
    COUNTERS["cublas"] += 1
    return torch.matmul(a, b)


def gemm_tn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    out = _native(a, b, "tn", None)
    if out is not None:
        return out
    COUNTERS["cublas"] += 1
    return torch.matmul(a.t(), b)


def gemm_tn_into(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[:] = a.T @ b`` where ``out`` may be a column slice of a larger row-major matrix."""
    if _BACKEND != "cublas":
        from . import gemm_tcgen05
        if gemm_tcgen05.supported(a, b, "tn") and out.stride(1) == 1 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0:
            COUNTERS["tcgen05"] += 1
            gemm_tcgen05.gemm(a, b, "tn", out=out)
            return out
    if _BACKEND != "cublas" and a.is_cuda and a.dtype == torch.bfloat16:
        from . import fallback
        if not fallback.vector_shaped(*a.shape, *b.shape):
            fallback.note("gemm", f"tn-into {tuple(a.shape)} x {tuple(b.shape)} out strides {out.stride()}")
    COUNTERS["cublas"] += 1
    torch.matmul(a.t(), b, out=out) if out.is_contiguous() else out.copy_(torch.matmul(a.t(), b))
    return out
