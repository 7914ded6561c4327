"""Python side of the tcgen05 GEMM (``csrc/gemm_tcgen05.cu``)."""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib


def supported(a: torch.Tensor, b: torch.Tensor, layout: str) -> bool:
    return False


def gemm(a, b, layout: str, bias: Optional[torch.Tensor]):
    raise _lib.NativeError("tcgen05 GEMM is not built")
